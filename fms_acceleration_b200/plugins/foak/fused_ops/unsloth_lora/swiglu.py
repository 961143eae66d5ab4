"""Names of fms_acceleration_foak/fused_ops/unsloth_lora/swiglu.py:40-98."""
from fms_acceleration_b200.ops.activation import glu_bwd, swiglu_fg_kernel  # noqa: F401


def swiglu_DWf_DW_dfg_kernel(DW, e, g):
    """Backward of ``h = silu(e) * g`` given ``DW = dL/dh``: returns ``(h, de, dg)`` (the reference writes them in
    place over ``DW``, ``e`` and ``g``; here they are new tensors)."""
    import torch

    h = torch.empty_like(e)
    de, dg = glu_bwd(DW, e, g, "silu", h_out=h)
    return h, de, dg
