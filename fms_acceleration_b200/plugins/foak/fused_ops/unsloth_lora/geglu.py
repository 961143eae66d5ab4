"""Names of fms_acceleration_foak/fused_ops/unsloth_lora/geglu.py:40-202."""
import torch

from fms_acceleration_b200.ops.activation import (geglu_approx_forward_kernel, geglu_exact_forward_kernel,  # noqa: F401
                                                  glu_bwd)


def geglu_exact_backward_kernel(DW, e, g):
    h = torch.empty_like(e)
    de, dg = glu_bwd(DW, e, g, "gelu", h_out=h)
    return h, de, dg


def geglu_approx_backward_kernel(DW, e, g):
    h = torch.empty_like(e)
    de, dg = glu_bwd(DW, e, g, "gelu_pytorch_tanh", h_out=h)
    return h, de, dg
