"""Products with a packed GPTQ weight under the reference's function names
(fms_acceleration_peft/gptqmodel/nn_modules/triton_utils/kernels.py:376-510).  The reference runs one Triton kernel
that unpacks tiles on the fly; here the weight goes through the CUDA dequantisation kernel and the tensor-core GEMM
(``ops/quant.py``, ``ops/gemm.py``), or through the fused few-rows kernel inside ``QuantLinear.forward``."""
from __future__ import annotations

import torch

from .dequant import QuantLinearFunction, dequant248  # noqa: F401
from .dequant import quant_matmul_248 as _matmul


def silu(x):
    return x * torch.sigmoid(x)


def quant_matmul_248(input, qweight, scales, qzeros, g_idx, bits, maxq):
    """``input [..., in] @ W [in, out]``."""
    return _matmul(input, qweight, scales, qzeros, g_idx, bits, maxq)


def transpose_quant_matmul_248(input, qweight, scales, qzeros, g_idx, bits, maxq):
    """``input [..., out] @ W^T``: the input gradient of :func:`quant_matmul_248`."""
    return _matmul(input, qweight, scales, qzeros, g_idx, bits, maxq, transpose=True)


def quant_matmul_inference_only_248(input, qweight, scales, qzeros, g_idx, bits, maxq):
    with torch.no_grad():
        return _matmul(input, qweight, scales, qzeros, g_idx, bits, maxq)


class QuantLinearInferenceOnlyFunction(torch.autograd.Function):
    """Forward only: nothing is saved and no gradient flows."""

    @staticmethod
    def forward(ctx, input, qweight, scales, qzeros, g_idx, bits, maxq):
        out = quant_matmul_inference_only_248(input, qweight, scales, qzeros, g_idx, bits, maxq)
        ctx.mark_non_differentiable(out)
        return out

    @staticmethod
    def backward(ctx, grad_output):  # pragma: no cover - stated for completeness
        raise RuntimeError("QuantLinearInferenceOnlyFunction has no backward")
