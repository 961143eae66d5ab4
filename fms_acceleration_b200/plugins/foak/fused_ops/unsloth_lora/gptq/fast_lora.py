"""Names of fms_acceleration_foak/fused_ops/unsloth_lora/gptq/fast_lora.py:19-859."""
from dataclasses import dataclass

import torch

from .._apply import LoRA_MLP, LoRA_QKV, LoRA_W, apply_lora_mlp, apply_lora_o, apply_lora_o_v2, apply_lora_qkv  # noqa: F401
from .triton.kernels import dequant248


@dataclass
class GPTQuantState:
    """The tensors of a GPTQ layer that a dequantisation needs."""

    qweight: torch.Tensor
    scales: torch.Tensor
    qzeros: torch.Tensor
    g_idx: torch.Tensor
    bits: int
    zero_offset: int = 0


def extract_gptq_state(qmodule) -> GPTQuantState:
    return GPTQuantState(qmodule.qweight, qmodule.scales, qmodule.qzeros, qmodule.g_idx, qmodule.bits,
                         getattr(qmodule, "zero_offset", 0))


def unpack_gptqstate(qstate: GPTQuantState):
    return qstate.qweight, qstate.scales, qstate.qzeros, qstate.g_idx, qstate.bits


def get_lora_parameters(proj):
    """``(quant state, A, B, scaling, dropout)`` of a LoRA-wrapped GPTQ projection."""
    from fms_acceleration_b200.ops.proj import _lora_parts, _unwrap

    base, lora = _unwrap(proj)
    qs = extract_gptq_state(base)
    if lora is None:
        return qs, None, None, None, None
    A, B, s = _lora_parts(lora)
    name = lora.active_adapters[0] if hasattr(lora, "active_adapters") else "default"
    return qs, A, B, s, (lora.lora_dropout[name] if hasattr(lora, "lora_dropout") else None)


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
