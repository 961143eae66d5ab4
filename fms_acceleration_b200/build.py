"""In-tree build of the native library (CUDA kernels for sm_100a + C++ host runtime).

``python -m fms_acceleration_b200.build`` compiles every ``csrc/*.cu`` and ``csrc/*.cpp`` into
object files under ``fms_acceleration_b200/lib/obj`` and links ``fms_acceleration_b200/lib/libfmsb200.so``.
Objects are rebuilt only when their source (or a header) is newer.  nvcc cross-compiles for
``sm_100a`` without a GPU present, so the build also serves as the "does it compile" check.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIBDIR = os.path.join(HERE, "lib")
OBJDIR = os.path.join(LIBDIR, "obj")
LIBNAME = "libfmsb200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-Wno-unused-function",
]
CXX_FLAGS = ["-O3", "-std=c++17", "-fPIC", "-pthread"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC or put it on PATH")


def _newest_header_mtime() -> float:
    m = 0.0
    for f in os.listdir(CSRC):
        if f.endswith((".cuh", ".h", ".hpp")):
            m = max(m, os.path.getmtime(os.path.join(CSRC, f)))
    return m


def library_path() -> str:
    return os.path.join(LIBDIR, LIBNAME)


def sources() -> list[str]:
    return sorted(f for f in os.listdir(CSRC) if f.endswith((".cu", ".cpp")))


def _compile_one(src: str, verbose: bool, ptxas_info: bool) -> str:
    obj = os.path.join(OBJDIR, os.path.splitext(src)[0] + ".o")
    path = os.path.join(CSRC, src)
    stamp = max(os.path.getmtime(path), _newest_header_mtime())
    if os.path.exists(obj) and os.path.getmtime(obj) >= stamp:
        return obj
    if src.endswith(".cu"):
        cmd = [_nvcc(), *NVCC_FLAGS, *os.environ.get("FMSB_NVCC_EXTRA", "").split(), "-I", CSRC, "-c", path, "-o", obj]
        if ptxas_info:
            cmd[1:1] = ["-Xptxas", "-v"]
    else:
        cmd = [os.environ.get("CXX", "g++"), *CXX_FLAGS, "-I", CSRC, "-c", path, "-o", obj]
    if verbose:
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"compiling {src} failed:\n{res.stdout}\n{res.stderr}")
    if ptxas_info and res.stderr:
        print(res.stderr)
    return obj


def build(verbose: bool = False, force: bool = False, ptxas_info: bool = False) -> str:
    """Compile and link the native library; returns its path."""
    os.makedirs(OBJDIR, exist_ok=True)
    if force:
        for f in os.listdir(OBJDIR):
            os.remove(os.path.join(OBJDIR, f))
    srcs = sources()
    with ThreadPoolExecutor(max_workers=min(8, max(1, len(srcs)))) as pool:
        objs = list(pool.map(lambda s: _compile_one(s, verbose, ptxas_info), srcs))
    lib = library_path()
    if force or not os.path.exists(lib) or any(os.path.getmtime(o) > os.path.getmtime(lib) for o in objs):
        cmd = [_nvcc(), "-shared", "-o", lib, *objs, "-lcudart", "-Xlinker", "--no-as-needed"]
        if verbose:
            print(" ".join(cmd), flush=True)
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"linking failed:\n{res.stdout}\n{res.stderr}")
    return lib


if __name__ == "__main__":
    out = build(verbose="-v" in sys.argv, force="--force" in sys.argv, ptxas_info="--ptxas" in sys.argv)
    print(out)
