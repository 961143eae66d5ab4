"""Kernel micro-benchmarks (``python -m fms_acceleration_b200.benchmarks.kernels --help``)."""
