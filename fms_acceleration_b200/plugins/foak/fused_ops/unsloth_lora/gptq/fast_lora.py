"""Names of fms_acceleration_foak/fused_ops/unsloth_lora/gptq/fast_lora.py:19-859."""
from dataclasses import dataclass
from typing import Optional

import torch

from .._apply import LoRA_MLP, LoRA_QKV, LoRA_W, apply_lora_mlp, apply_lora_o, apply_lora_o_v2, apply_lora_qkv  # noqa: F401
from .triton.kernels import dequant248


@dataclass
class GPTQuantState:
    """The tensors and sizes of a GPTQ layer (field names of the reference's state,
    fused_ops/unsloth_lora/gptq/fast_lora.py:20-45; the switches of other GPTQ back-ends are carried with their
    defaults).  ``zero_offset`` is the constant the stored zero points are short of the true ones (1 for the v1
    checkpoint format, 0 for v2)."""

    qweight: torch.Tensor
    scales: torch.Tensor
    qzeros: torch.Tensor
    g_idx: torch.Tensor
    bits: int
    zero_offset: int = 0
    infeatures: Optional[int] = None
    outfeatures: Optional[int] = None
    group_size: Optional[int] = None
    maxq: Optional[int] = None
    kernel_switch_threshold: Optional[int] = None
    autogptq_cuda_available: bool = False
    autogptq_cuda: bool = False
    wf: Optional[torch.Tensor] = None
    use_cuda_fp16: bool = False
    bias: Optional[torch.Tensor] = None
    trainable: bool = True


def _nonzero_bias(qmodule):
    bias = getattr(qmodule, "bias", None)
    return bias if bias is not None and bool(bias.count_nonzero() > 0) else None


def extract_gptq_state(qmodule) -> GPTQuantState:
    qmodule = getattr(qmodule, "base_layer", qmodule)
    return GPTQuantState(qmodule.qweight, qmodule.scales, qmodule.qzeros, qmodule.g_idx, qmodule.bits,
                         getattr(qmodule, "zero_offset", 0), infeatures=qmodule.infeatures,
                         outfeatures=qmodule.outfeatures, group_size=qmodule.group_size,
                         maxq=getattr(qmodule, "maxq", 2 ** qmodule.bits - 1), bias=_nonzero_bias(qmodule))


def unpack_gptqstate(qstate: GPTQuantState):
    return qstate.qweight, qstate.scales, qstate.qzeros, qstate.g_idx, qstate.bits


def get_lora_parameters(proj):
    """``(quant state, bias, A, B, scaling, dropout)`` of a LoRA-wrapped GPTQ projection; the four adapter entries
    are None for a bare layer or when the adapter is disabled or merged (reference :94-116)."""
    from fms_acceleration_b200.ops.proj import _lora_parts, _unwrap

    base, lora = _unwrap(proj)
    qs = extract_gptq_state(base)
    bias = getattr(base, "bias", None)
    if lora is None or getattr(lora, "disable_adapters", False) or getattr(lora, "merged", False):
        return qs, bias, None, None, None, None
    A, B, s = _lora_parts(lora)
    name = lora.active_adapters[0] if hasattr(lora, "active_adapters") else "default"
    return qs, bias, A, B, s, (lora.lora_dropout[name] if hasattr(lora, "lora_dropout") else None)


def matmul_lora(X, W, A, B, s, out=None, dropout=None):
    """``X W + s (dropout(X) A^T) B^T`` with ``W`` the dequantised ``[in, out]`` weight."""
    y = X @ W.to(X.dtype)
    if A is not None:
        xd = dropout(X) if dropout is not None else X
        y = y + s * ((xd @ A.to(X.dtype).t()) @ B.to(X.dtype).t())
    return y


def matmul_lora_canonicalized(X, W, A, B, s, dropout=None):
    """``X W + s (d(X) A^T) B^T`` for a rank-2 ``X [rows, in]`` and ``W [in, out]``; ``dropout`` is a mask tensor that
    multiplies ``X`` or a dropout module (the dropped-out input is left on it as ``dropout.X`` for the backward, as
    in the reference, fused_ops/unsloth_lora/gptq/fast_lora.py:119-140)."""
    out = X @ W.to(X.dtype)
    if dropout is not None:
        if isinstance(dropout, torch.Tensor):
            X = X * dropout
        elif isinstance(dropout, torch.nn.Module):
            X = dropout(X)
            dropout.X = X
        else:
            raise NotImplementedError("dropout must be a tensor or module.")
    return out + (X @ A.to(X.dtype).t()) @ (s * B.to(X.dtype).t())


def dequantize(qstate: GPTQuantState) -> torch.Tensor:
    return dequant248(qstate.qweight, qstate.scales, qstate.qzeros, qstate.g_idx, qstate.bits,
                      zero_offset=qstate.zero_offset)
