"""Step timing, NVTX ranges and roofline arithmetic.

The reference has no profiler or timers of its own; its throughput numbers are the Hugging Face trainer's
``train_tokens_per_second`` scraped from stdout (scripts/benchmarks/benchmark.py:539-568).  Here:

* :class:`StepTimer` times steps with CUDA events on the launching stream and reduces with a maximum over the ranks;
* :func:`nvtx_range` marks a region for a timeline profiler (a no-op without CUDA);
* :func:`roofline` turns (FLOPs, HBM bytes, NVLink bytes, measured milliseconds) into achieved rates and the fraction
  of the measured peaks (a cuBLAS bf16 GEMM and a device copy measured on the same kind of GPU, stored in
  ``MEASURED_PEAKS.json`` at the repository root; documented fallbacks otherwise).
"""
from __future__ import annotations

import contextlib
import json
import os
import time
from typing import Dict, List, Optional

import torch

_REPO_ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), "..", ".."))
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}
NVLINK_GBS_PER_DIRECTION = 770.0  # measured peer copy, per direction per GPU (900 nominal)


def measured_peaks(path: Optional[str] = None) -> Dict[str, float]:
    """Denominators of every roofline fraction: measured copy bandwidth and cuBLAS bf16 throughput."""
    path = path or os.path.join(_REPO_ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path, encoding="utf-8") as fh:
            raw = json.load(fh)
    except (OSError, ValueError):
        return dict(FALLBACK_PEAKS)
    out = dict(FALLBACK_PEAKS)
    for k in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained"):
        v = raw.get(k)
        if isinstance(v, dict):
            v = v.get("value")
        if isinstance(v, (int, float)) and v > 0:
            out[k] = float(v)
    out["source"] = "measured"
    return out


def roofline(ms: float, flops: float = 0.0, hbm_bytes: float = 0.0, nvlink_bytes: float = 0.0, sustained: bool = False,
             peaks: Optional[Dict[str, float]] = None) -> Dict[str, float]:
    """Achieved rates and the fraction of the roofline.

    The target time is the slowest of FLOPs / GEMM peak, HBM bytes / copy bandwidth and NVLink bytes / link
    bandwidth; ``fraction`` = target / measured.  ``sustained`` selects the power-capped GEMM figure, which is the right
    denominator for a kernel timed inside a long training step.
    """
    pk = peaks or measured_peaks()
    tf = pk["bf16_tflops_sustained" if sustained else "bf16_tflops"]
    t_flops = flops / (tf * 1e12) * 1e3
    t_hbm = hbm_bytes / (pk["hbm_gbs"] * 1e9) * 1e3
    t_link = nvlink_bytes / (NVLINK_GBS_PER_DIRECTION * 1e9) * 1e3
    target = max(t_flops, t_hbm, t_link)
    bound = "compute" if target == t_flops else ("hbm" if target == t_hbm else "nvlink")
    return {"ms": ms, "tflops": flops / ms / 1e9 if ms else 0.0, "hbm_gbs": hbm_bytes / ms / 1e6 if ms else 0.0,
            "nvlink_gbs": nvlink_bytes / ms / 1e6 if ms else 0.0, "target_ms": target, "bound": bound,
            "fraction": target / ms if ms else 0.0, "of": pk["source"]}


@contextlib.contextmanager
def nvtx_range(name: str):
    on = torch.cuda.is_available()
    if on:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if on:
            torch.cuda.nvtx.range_pop()


class StepTimer:
    """``with timer.step(): ...`` per training step; ``summary()`` gives the mean and the max over ranks.

    On a GPU each step is bracketed by CUDA events on the current stream (no synchronisation inside the step; the
    events are read in ``summary``).  On the CPU the wall clock is used.
    """

    def __init__(self, skip_first: int = 0):
        self.skip_first = skip_first
        self._events: List[tuple] = []
        self._wall: List[float] = []
        self.cuda = torch.cuda.is_available()

    @contextlib.contextmanager
    def step(self):
        if self.cuda:
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            try:
                yield
            finally:
                e.record()
                self._events.append((s, e))
        else:
            t0 = time.perf_counter()
            try:
                yield
            finally:
                self._wall.append((time.perf_counter() - t0) * 1e3)

    def times_ms(self) -> List[float]:
        if self.cuda:
            torch.cuda.synchronize()
            ts = [s.elapsed_time(e) for s, e in self._events]
        else:
            ts = list(self._wall)
        return ts[self.skip_first:]

    def summary(self, group=None) -> Dict[str, float]:
        ts = self.times_ms()
        mean = sum(ts) / len(ts) if ts else 0.0
        out = {"steps": len(ts), "mean_ms": mean, "min_ms": min(ts) if ts else 0.0, "max_ms": max(ts) if ts else 0.0}
        import torch.distributed as dist

        if dist.is_available() and dist.is_initialized():
            dev = torch.device("cuda", torch.cuda.current_device()) if self.cuda else torch.device("cpu")
            t = torch.tensor([mean], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
            out["mean_ms_max_over_ranks"] = float(t[0])
        return out
