"""GPTQ ``QuantLinear``: 2/4/8-bit packed weight with per-group scales and zero points.

Tensor layout is the GPTQ checkpoint layout the reference loads
(fms_acceleration_peft/gptqmodel/nn_modules/qlinear/qlinear_tritonv2.py:34-165): ``qweight`` int32
``[in*bits/32, out]`` (consecutive input rows packed along the bit positions), ``qzeros`` int32
``[groups, out*bits/32]`` (packed along the output columns), ``scales`` ``[groups, out]``, ``g_idx`` int32
``[in]``, optional ``bias``.  ``forward`` is dequantise (``csrc/quant.cu``) followed by the tcgen05 GEMM with
the dequantised ``[in, out]`` matrix as the MN-major operand, so no transpose is ever materialised; with few rows
(generation, evaluation of short prompts) int4 weights are expanded inside the GEMM instead
(``csrc/gemm_q4_fused.cu``, the counterpart of gptqmodel/nn_modules/triton_utils/kernels.py:105-201).
"""
from __future__ import annotations

import math

import torch
from torch import nn

from ..ops import quant as Q
from ..ops.gemm import FUSED_Q4_MAX_ROWS, gemm, gemm_gptq_fused


class QuantLinear(nn.Module):
    QUANT_TYPE = "b200"
    SUPPORTED_BITS = (2, 4, 8)
    SUPPORTED_GROUP_SIZE = ()          # empty: any group size (-1 = one group per column)
    SUPPORTED_DESC_ACT = (True, False)
    SUPPORTED_SYM = (True, False)
    SUPPORTED_SHARDS = True

    @classmethod
    def validate(cls, bits: int, group_size: int, desc_act: bool, sym: bool, raise_error: bool = True) -> bool:
        """Whether this layer can hold a weight quantised with these settings (the check the reference's
        ``BaseQuantLinear.validate`` makes before a kernel class is chosen,
        fms_acceleration_peft/gptqmodel/nn_modules/qlinear/__init__.py:16-43)."""
        err = None
        if bits not in cls.SUPPORTED_BITS:
            err = f"{cls.QUANT_TYPE} only supports {cls.SUPPORTED_BITS} bits: actual bits = {bits}"
        elif cls.SUPPORTED_GROUP_SIZE and group_size not in cls.SUPPORTED_GROUP_SIZE:
            err = f"{cls.QUANT_TYPE} only supports group sizes {cls.SUPPORTED_GROUP_SIZE}: actual group_size = {group_size}"
        elif sym not in cls.SUPPORTED_SYM:
            err = f"{cls.QUANT_TYPE} does not support sym = {sym}"
        elif desc_act not in cls.SUPPORTED_DESC_ACT:
            err = f"{cls.QUANT_TYPE} does not support desc_act = {desc_act}"
        if err is not None and raise_error:
            raise NotImplementedError(err)
        return err is None

    def __init__(self, bits: int, group_size: int, infeatures: int, outfeatures: int, bias: bool = False,
                 dtype: torch.dtype = torch.float16, zero_offset: int = 0, device=None, **kwargs):
        super().__init__()
        if bits not in self.SUPPORTED_BITS:
            raise NotImplementedError(f"bits={bits}: only {self.SUPPORTED_BITS} are supported")
        per = 32 // bits
        if infeatures % per != 0 or outfeatures % per != 0:
            raise NotImplementedError(f"in_features and out_features must be divisible by {per}")
        self.bits = bits
        self.group_size = group_size if group_size != -1 else infeatures
        self.infeatures = self.in_features = infeatures
        self.outfeatures = self.out_features = outfeatures
        self.maxq = 2 ** bits - 1
        self.zero_offset = zero_offset  # 1 for checkpoints in the v1 format (zero point stored minus one)
        groups = math.ceil(infeatures / self.group_size)
        self.register_buffer("qweight", torch.zeros(infeatures * bits // 32, outfeatures, dtype=torch.int32, device=device))
        self.register_buffer("qzeros", torch.zeros(groups, outfeatures * bits // 32, dtype=torch.int32, device=device))
        self.register_buffer("scales", torch.zeros(groups, outfeatures, dtype=dtype, device=device))
        self.register_buffer("g_idx", (torch.arange(infeatures, device=device) // self.group_size).to(torch.int32))
        if bias:
            self.register_buffer("bias", torch.zeros(outfeatures, dtype=dtype, device=device))
        else:
            self.bias = None
        self.compute_dtype = dtype
        self._sequential_groups = True

    @property
    def weight(self):
        return self.qweight

    def post_init(self):
        expected = (torch.arange(self.infeatures, device=self.g_idx.device) // self.group_size).to(torch.int32)
        self._sequential_groups = bool(torch.equal(self.g_idx, expected))

    # ------------------------------------------------------------------ packing
    def pack(self, linear: nn.Module, scales: torch.Tensor, zeros: torch.Tensor, g_idx: torch.Tensor | None = None):
        """Pack a float ``linear`` given per-group ``scales`` / ``zeros`` of shape [out, groups]."""
        W = linear.weight.data.float()  # [out, in]
        g = (g_idx if g_idx is not None else self.g_idx).long().to(W.device)
        sc = scales.t().contiguous().float().to(W.device)  # [groups, out]
        zp = zeros.t().contiguous().float().to(W.device)
        q = torch.round(W.t() / sc[g] + zp[g]).clamp_(0, self.maxq).to(torch.int64)  # [in, out]
        self.qweight = Q.gptq_pack(q, self.bits).to(self.qweight.device)
        self.qzeros = Q.gptq_pack_zeros((zp - self.zero_offset).round().to(torch.int64), self.bits).to(self.qzeros.device)
        self.scales = sc.to(self.scales.dtype).to(self.scales.device)
        self.g_idx = g.to(torch.int32).to(self.g_idx.device)
        if getattr(linear, "bias", None) is not None and self.bias is not None:
            self.bias = linear.bias.data.to(self.scales.dtype).to(self.scales.device)
        self.post_init()

    @classmethod
    def random(cls, infeatures, outfeatures, bits=4, group_size=128, dtype=torch.float16, device=None, generator=None,
               scale_std=0.002):
        """Random codes uniform in [0, 2^bits), scales ~ |normal(0, scale_std)|, symmetric zero point."""
        m = cls(bits, group_size, infeatures, outfeatures, False, dtype, 0, device)
        dev = m.qweight.device
        m.qweight = torch.randint(-2 ** 31, 2 ** 31 - 1, m.qweight.shape, dtype=torch.int32, device=dev, generator=generator)
        zp = torch.full((m.qzeros.shape[0], outfeatures), 2 ** (bits - 1), dtype=torch.int64, device=dev)
        m.qzeros = Q.gptq_pack_zeros(zp, bits)
        m.scales = (torch.randn(m.scales.shape, device=dev, generator=generator) * scale_std).abs().to(dtype)
        return m

    # ------------------------------------------------------------------ compute
    def dequantize(self, out=None, dtype=None) -> torch.Tensor:
        """Dense ``[in, out]`` weight."""
        scales = self._scales_as(dtype)
        g_idx = None if self._sequential_groups else self.g_idx
        return Q.gptq_dequant(self.qweight, scales, self.qzeros, g_idx if self.qweight.is_cuda else self.g_idx,
                              self.bits, self.group_size, self.zero_offset, out=out)

    def _scales_as(self, dtype) -> torch.Tensor:
        if dtype is None or dtype == self.scales.dtype:
            return self.scales
        cached = getattr(self, "_scales_cast", None)
        if cached is None or cached[0] != dtype or cached[1] is not self.scales:
            cached = (dtype, self.scales, self.scales.to(dtype))  # the weights are frozen: convert once
            self._scales_cast = cached
        return cached[2]

    def fused_ok(self, x: torch.Tensor) -> bool:
        """Few rows, int4, groups in order and a multiple of 64 wide: dequantise inside the GEMM."""
        rows = x.numel() // x.shape[-1]
        return (x.is_cuda and x.dtype in (torch.float16, torch.bfloat16) and self.bits == 4 and rows <= FUSED_Q4_MAX_ROWS
                and self._sequential_groups and self.group_size % 64 == 0 and self.infeatures % self.group_size == 0
                and self.infeatures % 64 == 0)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.fused_ok(x):
            y = _GPTQFusedMatmul.apply(x, self)
            return y if self.bias is None else y + self.bias.to(y.dtype)
        w = self.dequantize(dtype=x.dtype if x.dtype in (torch.float16, torch.bfloat16) else None)
        if x.is_cuda and x.dtype in (torch.float16, torch.bfloat16):
            y = _GPTQMatmul.apply(x, w)
        else:
            y = x @ w.to(x.dtype)
        if self.bias is not None:
            y = y + self.bias.to(y.dtype)
        return y

    @classmethod
    def warmup(cls, model, transpose: bool = False, seqlen: int = 2048) -> int:
        """The reference pre-tunes its Triton kernel for every distinct ``(in, out)`` shape here
        (gptqmodel/nn_modules/qlinear/qlinear_tritonv2.py:184-230); these kernels choose their tiles from the problem
        size, so there is nothing to tune.  Returns the number of distinct shapes found."""
        return len({(m.infeatures, m.outfeatures) for m in model.modules() if isinstance(m, cls)})

    def extra_repr(self):
        return f"in={self.infeatures}, out={self.outfeatures}, bits={self.bits}, group_size={self.group_size}"


class _GPTQFusedMatmul(torch.autograd.Function):
    """Forward through the fused int4 dequantise+GEMM kernel (few rows); the backward (dx only) expands the weight."""

    @staticmethod
    def forward(ctx, x, layer):
        ctx.layer, ctx.shape = layer, x.shape
        x2 = x.reshape(-1, x.shape[-1])
        if x2.stride(1) != 1 or x2.stride(0) % 8:
            x2 = x2.contiguous()
        y = gemm_gptq_fused(x2, layer.qweight, layer._scales_as(x.dtype), layer.qzeros, layer.group_size,
                            layer.zero_offset)
        return y.view(*x.shape[:-1], layer.outfeatures)

    @staticmethod
    def backward(ctx, dy):
        dy2 = dy.reshape(-1, dy.shape[-1])
        if dy2.stride(1) != 1 or dy2.stride(0) % 8:
            dy2 = dy2.contiguous()
        w = ctx.layer.dequantize(dtype=dy.dtype)
        return gemm(dy2, w).view(ctx.shape), None


class _GPTQMatmul(torch.autograd.Function):
    """y = x W for a frozen dequantised ``W [in, out]``; backward is ``dy W^T`` (cf. ``QuantLinearFunction``,
    fms_acceleration_peft/gptqmodel/nn_modules/triton_utils/dequant.py:141-161)."""

    @staticmethod
    def forward(ctx, x, w):
        ctx.save_for_backward(w)
        ctx.shape = x.shape
        y = gemm(x.reshape(-1, x.shape[-1]), w, b_mn=True)
        return y.view(*x.shape[:-1], w.shape[1])

    @staticmethod
    def backward(ctx, dy):
        (w,) = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if dy2.stride(1) != 1 or dy2.stride(0) % 8:
            dy2 = dy2.contiguous()
        return gemm(dy2, w).view(ctx.shape), None
