"""Fused ops and kernels plugin."""
from .framework_plugin_fast_kernels import FastKernelsAccelerationPlugin  # noqa: F401
