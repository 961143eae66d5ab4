"""The reference's module path for its vendored ScatterMoE operators (scattermoe_utils/khd/).  The operators of that
name are stated here over this package's own primitives; the training path (``ScatterMoE.forward``) goes through
``ops/moe.py`` and the grouped tensor-core GEMM instead."""
from .custom_op import torch_custom_op  # noqa: F401,E402
