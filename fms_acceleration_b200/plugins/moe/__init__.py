"""Accelerated mixture-of-experts: ScatterMoE modules on grouped tcgen05 GEMMs, expert parallelism, checkpoint tools."""
from .framework_plugin_scattermoe import ScatterMoEAccelerationPlugin  # noqa: F401
