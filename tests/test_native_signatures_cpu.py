"""Every ctypes signature registered in Python against the `extern "C"` definition it binds: same number of
parameters, pointers where the C side takes pointers, 64-bit integers where it takes `long long`.  A mismatch would
corrupt arguments silently at call time; this catches it without a GPU."""
import ctypes
import importlib
import os
import pkgutil
import re

import fms_acceleration_b200
from fms_acceleration_b200 import _native as NV

CSRC = os.path.join(os.path.dirname(fms_acceleration_b200.__file__), "csrc")


def _c_definitions():
    """name -> list of parameter type strings, from the sources."""
    defs = {}
    pat = re.compile(r'extern\s+"C"\s+[\w\s\*]+?\b(fmsb_\w+)\s*\(([^)]*)\)\s*\{', re.S)
    for f in sorted(os.listdir(CSRC)):
        if not f.endswith((".cu", ".cpp")):
            continue
        src = open(os.path.join(CSRC, f), encoding="utf-8").read()
        src = re.sub(r"//[^\n]*", "", src)
        for m in pat.finditer(src):
            params = [p.strip() for p in m.group(2).replace("\n", " ").split(",") if p.strip()]
            if params == ["void"]:
                params = []
            defs[m.group(1)] = params
    return defs


def _import_all_modules():
    for mod in pkgutil.walk_packages(fms_acceleration_b200.__path__, fms_acceleration_b200.__name__ + "."):
        if ".csrc" in mod.name or mod.name.endswith(".build"):
            continue
        try:
            importlib.import_module(mod.name)
        except Exception:  # optional dependencies
            pass


def _kind(ctype):
    if ctype in (ctypes.c_void_p, ctypes.c_char_p) or (isinstance(ctype, type) and issubclass(ctype, ctypes._Pointer)):
        return "ptr"
    if ctype in (ctypes.c_longlong, ctypes.c_ulonglong, ctypes.c_int64, ctypes.c_uint64, ctypes.c_size_t):
        return "i64"
    if ctype in (ctypes.c_float,):
        return "f32"
    if ctype in (ctypes.c_double,):
        return "f64"
    return "i32"


def _c_kind(param: str):
    p = param.split("=")[0].strip()
    if "*" in p or "cudaStream_t" in p:
        return "ptr"
    if re.search(r"\blong long\b|\bint64_t\b|\buint64_t\b|\bsize_t\b", p):
        return "i64"
    if re.search(r"\bfloat\b", p):
        return "f32"
    if re.search(r"\bdouble\b", p):
        return "f64"
    return "i32"


def test_python_signatures_match_the_c_definitions():
    _import_all_modules()
    defs = _c_definitions()
    assert len(defs) > 40, "the source scan found too few entry points"
    checked = 0
    for name, argtypes in NV._SIGNATURES.items():
        assert name in defs, f"{name} is declared in Python but not defined in csrc"
        c_params = defs[name]
        assert len(argtypes) == len(c_params), (name, len(argtypes), c_params)
        for i, (a, c) in enumerate(zip(argtypes, c_params)):
            assert _kind(a) == _c_kind(c), (name, i, a, c)
        checked += 1
    assert checked > 40
