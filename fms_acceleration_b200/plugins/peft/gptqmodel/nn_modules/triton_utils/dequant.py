"""``dequant248`` and ``quant_matmul_248`` with the reference's argument order
(fms_acceleration_peft/gptqmodel/nn_modules/triton_utils/dequant.py:103-161)."""
from __future__ import annotations

import torch

from fms_acceleration_b200.ops import quant as Q
from fms_acceleration_b200.ops.gemm import gemm


def dequant248(qweight, scales, qzeros, g_idx, bits: int, maxq=None, zero_offset: int = 0) -> torch.Tensor:
    """Dense ``[in, out]`` weight in the dtype of ``scales``."""
    group_size = qweight.shape[0] * 32 // bits // scales.shape[0]
    if not qweight.is_cuda:
        return Q.gptq_dequant_ref(qweight, scales, qzeros, g_idx, bits, zero_offset).to(scales.dtype)
    return Q.gptq_dequant(qweight, scales, qzeros, g_idx, bits, group_size, zero_offset)


def quant_matmul_248(input, qweight, scales, qzeros, g_idx, bits: int, maxq=None, transpose: bool = False):
    """``input @ W`` (or ``input @ W^T`` with ``transpose``) through the dequantised weight; the weight takes no
    gradient."""
    W = dequant248(qweight, scales, qzeros, g_idx, bits)
    x2 = input.reshape(-1, input.shape[-1])
    if x2.is_cuda and x2.dtype in (torch.float16, torch.bfloat16):
        y = gemm(x2.contiguous(), W.to(x2.dtype), b_mn=not transpose)
    else:
        y = x2 @ (W.t() if transpose else W).to(x2.dtype)
    return y.reshape(*input.shape[:-1], y.shape[-1])


class QuantLinearFunction(torch.autograd.Function):
    """``input @ W`` for a packed GPTQ weight with the reference's argument list (dequant.py:141-161): the weight is
    expanded for the product and again, transposed, for the input gradient; the packed tensors take no gradient."""

    @staticmethod
    def forward(ctx, input, qweight, scales, qzeros, g_idx, bits, maxq):
        ctx.save_for_backward(qweight, scales, qzeros, g_idx)
        ctx.bits, ctx.maxq = bits, maxq
        return quant_matmul_248(input, qweight, scales, qzeros, g_idx, bits, maxq)

    @staticmethod
    def backward(ctx, grad_output):
        qweight, scales, qzeros, g_idx = ctx.saved_tensors
        grad_input = None
        if ctx.needs_input_grad[0]:
            grad_input = quant_matmul_248(grad_output, qweight, scales, qzeros, g_idx, ctx.bits, ctx.maxq, transpose=True)
        return grad_input, None, None, None, None, None, None
