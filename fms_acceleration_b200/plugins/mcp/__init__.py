"""Mamba context parallelism."""
from .framework_plugin_mcp import MCPAccelerationPlugin  # noqa: F401
