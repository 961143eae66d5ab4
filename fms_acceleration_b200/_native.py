"""ctypes binding to the in-tree native library ``lib/libfmsb200.so``.

Every native entry point is an ``extern "C"`` launcher taking raw device pointers, sizes and a
``cudaStream_t``; the Python wrappers in :mod:`fms_acceleration_b200.ops` own allocation and autograd.
The library is built in-tree (see :mod:`fms_acceleration_b200.build`); on a machine with a GPU a
missing library is an error, never a silent fallback.
"""
from __future__ import annotations

import ctypes
import os
import threading
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

_LIB = None
_LOCK = threading.Lock()

P = c_void_p
I = c_int
L = c_longlong
F = c_float

# name -> argtypes (all return int)
_SIGNATURES = {
    "fmsb_gemm": [P, L, P, L, I, P, L, P, L, I, I, I, P, L, I, P, L, F, F, I, I, I, I, I, P, P],
    "fmsb_rmsnorm_fwd": [P, P, P, P, P, P, I, I, F, I, I, P],
    "fmsb_rmsnorm_bwd": [P, P, P, P, P, P, P, P, I, I, I, I, I, P],
    "fmsb_rope": [P, P, P, P, I, I, I, L, F, I, P],
    "fmsb_glu_fwd": [P, P, P, I, I, L, L, L, I, I, P, P],
    "fmsb_glu_bwd": [P, P, P, P, P, P, I, I, L, L, L, L, L, L, I, I, P, P],
    "fmsb_add": [P, P, P, L, I, P],
    "fmsb_ce": [P, L, P, P, P, P, P, I, I, I, F, I, I, P],
    "fmsb_ce_bwd": [P, L, P, L, P, P, P, L, I, I, I, I, P],
    "fmsb_count_valid": [P, L, I, P, P],
    "fmsb_quant4": [P, L, P, I, P, P, I, P],
    "fmsb_quant8_blockwise": [P, L, F, P, P, P, P],
    "fmsb_dequant4": [P, P, P, P, P, F, P, I, L, P, I, P],
    "fmsb_gptq_dequant": [P, P, P, P, I, I, I, I, I, P, L, I, P],
}


def library_path() -> str:
    return os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib", "libfmsb200.so")


def available() -> bool:
    return os.path.exists(library_path())


def lib():
    """Load (once) and return the native library."""
    global _LIB
    if _LIB is not None:
        return _LIB
    with _LOCK:
        if _LIB is not None:
            return _LIB
        path = library_path()
        if not os.path.exists(path):
            raise RuntimeError(
                f"native library {path} is missing: run `python -m fms_acceleration_b200.build` "
                "(the CUDA kernels of this package have no PyTorch fallback on a GPU)"
            )
        handle = ctypes.CDLL(path)
        for name, argtypes in _SIGNATURES.items():
            try:
                fn = getattr(handle, name)
            except AttributeError:
                continue
            fn.argtypes = argtypes
            fn.restype = c_int
        _LIB = _CountingLib(handle)
    return _LIB


class _CountingLib:
    """Thin proxy over the CDLL handle that counts calls into the native launchers."""

    def __init__(self, handle):
        self._handle = handle
        self._cache = {}
        self.calls = 0

    def __getattr__(self, name):
        fn = self._cache.get(name)
        if fn is None:
            raw = getattr(self._handle, name)

            def fn(*args, _raw=raw):
                self.calls += 1
                return _raw(*args)

            self._cache[name] = fn
        return fn


def launch_count() -> int:
    """Number of native launcher calls made by this process so far."""
    return 0 if _LIB is None else _LIB.calls


def declare(name: str, argtypes) -> None:
    """Register the signature of an entry point defined outside this table."""
    _SIGNATURES[name] = argtypes
    if _LIB is not None and hasattr(_LIB._handle, name):
        fn = getattr(_LIB._handle, name)
        fn.argtypes = argtypes
        fn.restype = c_int


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def ptr(t) -> int | None:
    return None if t is None else t.data_ptr()


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float16:
        return 0
    if dt == torch.bfloat16:
        return 1
    if dt == torch.float32:
        return 2
    raise TypeError(f"unsupported dtype {dt}")


class NativeError(RuntimeError):
    pass


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise NativeError(f"{what} failed with code {rc}")


_STATUS_NAMES = {
    1: "TMA producer timed out waiting for a free stage",
    2: "MMA issuer timed out",
    3: "epilogue timed out waiting for an accumulator",
    4: "wait on a peer flag timed out",
    5: "bad argument detected on device",
    6: "dequant warps timed out",
}

_status_words: dict[int, torch.Tensor] = {}


def _peer_wait_units() -> int:
    """Budget of a device-side wait on another rank, in units of 2^20 SM cycles (``FMSB_PEER_WAIT_S`` seconds at a
    nominal 1.9 GHz, default 20 s: ranks drift apart while one saves a checkpoint or waits for its data)."""
    sec = float(os.environ.get("FMSB_PEER_WAIT_S", "20"))
    return max(1, int(sec * 1.9e9) >> 20)


def status_word(device=None) -> torch.Tensor:
    """Per-device status block (4 x int32) shared by all kernels with bounded waits: [0] the status code (0 = fine),
    [1] the budget of waits on other ranks in units of 2^20 cycles; the rest is reserved."""
    dev = torch.cuda.current_device() if device is None else torch.device(device).index
    if dev is None:
        dev = torch.cuda.current_device()
    w = _status_words.get(dev)
    if w is None:
        w = torch.tensor([0, _peer_wait_units(), 0, 0], dtype=torch.int32, device=f"cuda:{dev}")
        _status_words[dev] = w
    return w


def set_peer_wait(seconds: float, device=None) -> None:
    """Change the budget of device-side waits on other ranks (tests of the time-out path use a short one)."""
    status_word(device)[1] = max(1, int(seconds * 1.9e9) >> 20)


def check_status(device=None) -> None:
    """Synchronising check of the status word; raises if any kernel reported a time-out."""
    w = status_word(device)
    v = int(w[0].item())
    if v != 0:
        w[0] = 0
        raise NativeError(f"device status {v}: {_STATUS_NAMES.get(v, 'unknown')}")


class StatusMonitor:
    """Checks the status word once per step WITHOUT a host synchronisation: ``poll()`` (end of a step) enqueues a
    4-byte copy into pinned host memory and records an event; ``raise_if_set()`` (start of the next step) looks at
    the snapshot only if its event has completed, so the host never waits for the device.  A time-out is therefore
    raised at most one step late; the word is cleared when it is raised, because every bounded wait on the device
    gives up early while it is non-zero."""

    def __init__(self, device=None):
        self.word = status_word(device)
        self.host = torch.zeros(1, dtype=torch.int32).pin_memory()
        self.event = None

    def poll(self) -> None:
        self.host.copy_(self.word[:1], non_blocking=True)
        self.event = torch.cuda.Event()
        self.event.record(torch.cuda.current_stream(self.word.device))

    def raise_if_set(self, wait: bool = False) -> None:
        if self.event is None:
            return
        if wait:
            self.event.synchronize()
        elif not self.event.query():
            return
        self.event = None
        v = int(self.host[0])
        if v != 0:
            self.word[0] = 0
            raise NativeError(f"device status {v}: {_STATUS_NAMES.get(v, 'unknown')} (reported by an earlier step)")

declare("fmsb_attn_fwd", [P, L, P, L, P, L, P, L, P, P, P, I, I, I, I, F, I, P, P])
declare("fmsb_attn_delta", [P, P, L, L, P, I, I, I, I, P])
declare("fmsb_attn_bwd_dq3", [P, L, P, L, P, L, P, L, P, L, P, P, P, P, I, I, I, I, F, I, P, P])
declare("fmsb_attn_bwd_dkv3", [P, L, P, L, P, L, P, L, P, L, P, L, P, P, P, P, I, I, I, I, F, I, P, P])
