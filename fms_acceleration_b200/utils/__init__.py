"""Profiling, roofline and failure-detection helpers."""
from .profiling import StepTimer, measured_peaks, nvtx_range, roofline  # noqa: F401
