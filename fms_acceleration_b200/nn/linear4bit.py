"""``Linear4bit``: an ``nn.Linear`` replacement whose weight is stored 4-bit blockwise (NF4 / FP4) with
double-quantised block scales.

Plays the role of bitsandbytes' ``Linear4bit`` that the reference loads through
``BitsAndBytesConfig(load_in_4bit=True, bnb_4bit_use_double_quant=True, bnb_4bit_quant_type=...)``
(fms_acceleration_peft/framework_plugin_bnb.py:143-149).  All tensors of the quantised state are plain
buffers so that the sharded-parameter engine can shard and gather them as bytes.
"""
from __future__ import annotations

import torch
from torch import nn

from ..ops import quant as Q
from ..ops.gemm import FUSED_Q4_MAX_ROWS, gemm, gemm_q4_fused


class Linear4bit(nn.Module):
    def __init__(self, in_features: int, out_features: int, bias: bool = False, quant_type: str = "nf4",
                 blocksize: int = 64, compute_dtype: torch.dtype = torch.bfloat16, device=None):
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.quant_type = quant_type
        self.blocksize = blocksize
        self.compute_dtype = compute_dtype
        n = in_features * out_features
        nb = n // blocksize
        self.register_buffer("weight", torch.zeros(n // 2, dtype=torch.uint8, device=device))
        self.register_buffer("absmax_q", torch.zeros(nb, dtype=torch.uint8, device=device))
        self.register_buffer("absmax2", torch.zeros((nb + 255) // 256, dtype=torch.float32, device=device))
        self.register_buffer("code2", Q.dynamic_code_book(device))
        self.register_buffer("code", Q.code_book(quant_type, device))
        self.register_buffer("offset", torch.zeros((), dtype=torch.float32, device=device))
        self._offset_f: float | None = None
        if bias:
            self.bias = nn.Parameter(torch.zeros(out_features, dtype=compute_dtype, device=device))
        else:
            self.bias = None

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_linear(cls, lin: nn.Linear, quant_type="nf4", blocksize=64, compute_dtype=None) -> "Linear4bit":
        return cls.from_weight(lin.weight.data, lin.bias, quant_type, blocksize, compute_dtype or lin.weight.dtype)

    @classmethod
    def from_weight(cls, w: torch.Tensor, bias=None, quant_type="nf4", blocksize=64,
                    compute_dtype=torch.bfloat16) -> "Linear4bit":
        out_f, in_f = w.shape
        m = cls(in_f, out_f, bias is not None, quant_type, blocksize, compute_dtype, device=w.device)
        m.load_quant_state(Q.quantize_4bit(w, quant_type, blocksize, True, compute_dtype))
        if bias is not None:
            m.bias.data.copy_(bias.data)
        return m

    def load_quant_state(self, qs: Q.Quant4State) -> None:
        self.weight = qs.packed
        self.absmax_q = qs.absmax_q
        self.absmax2 = qs.absmax2
        self.code2 = qs.code2
        self.code = qs.code
        self.offset = torch.tensor(qs.offset, dtype=torch.float32, device=qs.packed.device)
        self._offset_f = float(qs.offset)

    def quant_state(self) -> Q.Quant4State:
        if self._offset_f is None:
            self._offset_f = float(self.offset.item())
        return Q.Quant4State(packed=self.weight, shape=(self.out_features, self.in_features),
                             quant_type=self.quant_type, blocksize=self.blocksize, absmax_q=self.absmax_q,
                             code2=self.code2, absmax2=self.absmax2, offset=self._offset_f, code=self.code,
                             dtype=self.compute_dtype)

    # ------------------------------------------------------------------ compute
    def dequantize(self, out: torch.Tensor | None = None, dtype=None) -> torch.Tensor:
        return Q.dequantize_4bit(self.quant_state(), dtype or self.compute_dtype, out=out)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        rows = x.numel() // max(1, x.shape[-1])
        if (x.is_cuda and x.dtype in (torch.bfloat16, torch.float16) and rows <= FUSED_Q4_MAX_ROWS
                and self.blocksize == 64 and self.in_features % 64 == 0 and self.out_features % 8 == 0):
            # few rows: the weight is streamed as 4-bit data and expanded inside the GEMM kernel
            y = _FusedQuantMatmul.apply(x, self)
            return y if self.bias is None else y + self.bias.to(y.dtype)
        w = self.dequantize(dtype=x.dtype if x.dtype in (torch.bfloat16, torch.float16) else None)
        if x.is_cuda and x.dtype in (torch.bfloat16, torch.float16):
            y = _QuantMatmul.apply(x, w)
        else:
            y = torch.nn.functional.linear(x, w.to(x.dtype))
        if self.bias is not None:
            y = y + self.bias.to(y.dtype)
        return y

    def extra_repr(self) -> str:
        return f"in={self.in_features}, out={self.out_features}, {self.quant_type}, blocksize={self.blocksize}"


class _FusedQuantMatmul(torch.autograd.Function):
    """Forward through the fused dequantise+GEMM kernel; the backward (dx only) expands the weight once."""

    @staticmethod
    def forward(ctx, x, layer):
        ctx.layer = layer
        ctx.shape = x.shape
        x2 = x.reshape(-1, x.shape[-1])
        if x2.stride(1) != 1 or x2.stride(0) % 8:
            x2 = x2.contiguous()
        y = gemm_q4_fused(x2, layer.quant_state())
        return y.view(*x.shape[:-1], layer.out_features)

    @staticmethod
    def backward(ctx, dy):
        dy2 = dy.reshape(-1, dy.shape[-1])
        if dy2.stride(1) != 1 or dy2.stride(0) % 8:
            dy2 = dy2.contiguous()
        w = ctx.layer.dequantize(dtype=dy.dtype)
        return gemm(dy2, w, b_mn=True).view(ctx.shape), None


class _QuantMatmul(torch.autograd.Function):
    """y = x W^T with a frozen dense ``W``; only dx is produced."""

    @staticmethod
    def forward(ctx, x, w):
        ctx.save_for_backward(w)
        ctx.shape = x.shape
        y = gemm(x.reshape(-1, x.shape[-1]), w)
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        (w,) = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if dy2.stride(1) != 1 or dy2.stride(0) % 8:
            dy2 = dy2.contiguous()
        dx = gemm(dy2, w, b_mn=True)
        return dx.view(ctx.shape), None
