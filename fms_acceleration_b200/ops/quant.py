"""4-bit blockwise weights (NF4 / FP4 with double-quantised block scales) and GPTQ packed weights.

The formats follow what the reference consumes through bitsandbytes
(fms_acceleration_foak/fused_ops/unsloth_lora/utils.py:86-141: 8-bit block scales are expanded with a
256-entry code book and a per-256 scale, an ``offset`` is added, then the packed nibbles are expanded with
the 16-entry code book and multiplied by the block scale) and through its GPTQ kernels
(fms_acceleration_foak/fused_ops/unsloth_lora/gptq/triton/kernels.py:15-40).  Code books are data carried
with the weight, so any 16-entry / 256-entry table is supported.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import _native as N

# 16 quantiles of a standard normal, rescaled to [-1, 1] with an exact zero (the "NormalFloat4" data type
# of the QLoRA paper, Dettmers et al. 2023, appendix E).
NF4_CODE = [
    -1.0, -0.6961928009986877, -0.5250730514526367, -0.39491748809814453, -0.28444138169288635,
    -0.18477343022823334, -0.09105003625154495, 0.0, 0.07958029955625534, 0.16093020141124725,
    0.24611230194568634, 0.33791524171829224, 0.44070982933044434, 0.5626170039176941, 0.7229568362236023, 1.0,
]
# 4-bit float with 1 sign, 2 exponent and 1 mantissa bit, normalised to a maximum of 1; index bit 3 is the sign.
FP4_CODE = [
    0.0, 0.0625 / 12.0, 8.0 / 12.0, 1.0, 4.0 / 12.0, 6.0 / 12.0, 2.0 / 12.0, 3.0 / 12.0,
    -0.0, -0.0625 / 12.0, -8.0 / 12.0, -1.0, -4.0 / 12.0, -6.0 / 12.0, -2.0 / 12.0, -3.0 / 12.0,
]


def code_book(quant_type: str, device=None) -> torch.Tensor:
    if quant_type == "nf4":
        vals = NF4_CODE
    elif quant_type == "fp4":
        vals = FP4_CODE
    else:
        raise ValueError(f"unknown 4-bit type {quant_type!r}")
    return torch.tensor(vals, dtype=torch.float32, device=device)


_CODE_BOOKS: dict = {}


def dynamic_code_book(device=None, exponent_bits: int = 7, total_bits: int = 8) -> torch.Tensor:
    """Sorted 256-entry signed "dynamic exponent" code book used for the 8-bit block scales: decade
    10^-(6-i) carries 2^i linearly spaced fractions between 0.1 and 1, plus the end points 0 and 1.
    Built once per (device, format) and shared by every quantised layer (the table is read-only)."""
    key = (str(torch.device(device)) if device is not None else "cpu", exponent_bits, total_bits)
    cached = _CODE_BOOKS.get(key)
    if cached is not None:
        return cached
    vals: list[float] = []
    value_bits = total_bits - 1
    for i in range(exponent_bits):
        n_frac = 2 ** (i + value_bits - exponent_bits) + 1
        edges = torch.linspace(0.1, 1.0, n_frac, dtype=torch.float64)
        mids = ((edges[:-1] + edges[1:]) / 2.0).tolist()
        scale = 10.0 ** (-(exponent_bits - 1) + i)
        vals += [scale * m for m in mids]
        vals += [-scale * m for m in mids]
    extra = 2 ** (value_bits - exponent_bits) - 1
    if extra > 0:
        edges = torch.linspace(0.1, 1.0, extra + 1, dtype=torch.float64)
        mids = ((edges[:-1] + edges[1:]) / 2.0).tolist()
        scale = 10.0 ** (-(exponent_bits - 1) + exponent_bits - 1)
        vals += [scale * m for m in mids]
        vals += [-scale * m for m in mids]
    vals += [0.0, 1.0]
    vals += [0.0] * (2 ** total_bits - len(vals))
    vals.sort()
    book = torch.tensor(vals, dtype=torch.float32, device=device)
    _CODE_BOOKS[key] = book
    return book


@dataclass
class Quant4State:
    """A 4-bit blockwise quantised tensor.  ``absmax`` holds fp32 block scales when the scales are not
    double-quantised; otherwise ``absmax_q`` (uint8), ``code2``, ``absmax2`` and ``offset`` describe them."""

    packed: torch.Tensor              # uint8 [numel/2]
    shape: tuple
    quant_type: str = "nf4"
    blocksize: int = 64
    absmax: torch.Tensor | None = None
    absmax_q: torch.Tensor | None = None
    code2: torch.Tensor | None = None
    absmax2: torch.Tensor | None = None
    offset: float = 0.0
    code: torch.Tensor | None = None
    dtype: torch.dtype = torch.bfloat16

    @property
    def numel(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n

    def to(self, device):
        kw = {}
        for f in ("packed", "absmax", "absmax_q", "code2", "absmax2", "code"):
            t = getattr(self, f)
            kw[f] = None if t is None else t.to(device)
        return Quant4State(shape=self.shape, quant_type=self.quant_type, blocksize=self.blocksize,
                           offset=self.offset, dtype=self.dtype, **kw)

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in
                   (self.packed, self.absmax, self.absmax_q, self.absmax2) if t is not None)


# ---------------------------------------------------------------------------------------- CPU oracle
def _quant4_ref(w: torch.Tensor, code: torch.Tensor, blocksize: int):
    flat = w.reshape(-1).float()
    n = flat.numel()
    nb = (n + blocksize - 1) // blocksize
    pad = nb * blocksize - n
    if pad:
        flat = torch.cat([flat, flat.new_zeros(pad)])
    blk = flat.view(nb, blocksize)
    absmax = blk.abs().amax(dim=1)
    inv = torch.where(absmax > 0, 1.0 / absmax, torch.zeros_like(absmax))
    norm = blk * inv[:, None]
    idx = (norm[..., None] - code.to(norm.device)[None, None, :]).abs().argmin(dim=-1).view(-1)[:n]
    packed = ((idx[0::2] << 4) | idx[1::2]).to(torch.uint8)
    return packed, absmax


def _quant8_ref(v: torch.Tensor, offset: float, code2: torch.Tensor):
    x = v.float() - offset
    n = x.numel()
    nb = (n + 255) // 256
    pad = nb * 256 - n
    xp = torch.cat([x, x.new_zeros(pad)]) if pad else x
    blk = xp.view(nb, 256)
    absmax2 = blk.abs().amax(dim=1)
    t = torch.where(absmax2[:, None] > 0, blk / absmax2[:, None], torch.zeros_like(blk)).reshape(-1)[:n]
    q = (t[:, None] - code2.to(t.device)[None, :]).abs().argmin(dim=-1).to(torch.uint8)
    return q, absmax2


def block_scales(qs: Quant4State) -> torch.Tensor:
    """fp32 block scales (expands the double quantisation)."""
    if qs.absmax_q is None:
        return qs.absmax
    nb = qs.absmax_q.numel()
    s2 = qs.absmax2.repeat_interleave(256)[:nb]
    return qs.code2[qs.absmax_q.long()] * s2 + qs.offset


def dequantize_4bit_ref(qs: Quant4State, dtype=None) -> torch.Tensor:
    dtype = dtype or qs.dtype
    code = qs.code if qs.code is not None else code_book(qs.quant_type, qs.packed.device)
    p = qs.packed.long()
    idx = torch.stack([p >> 4, p & 15], dim=1).reshape(-1)
    n = qs.numel
    s = block_scales(qs).repeat_interleave(qs.blocksize)[:n]
    return (code[idx[:n]] * s).to(dtype).view(qs.shape)


# ---------------------------------------------------------------------------------------- front-ends
def quantize_4bit(w: torch.Tensor, quant_type: str = "nf4", blocksize: int = 64, double_quant: bool = True,
                  dtype: torch.dtype | None = None) -> Quant4State:
    """Quantise ``w`` (any shape, numel a multiple of 32) blockwise to 4 bits."""
    dev = w.device
    code = code_book(quant_type, dev)
    n = w.numel()
    if n % 32 != 0:
        raise ValueError("numel must be a multiple of 32")
    if w.is_cuda:
        wc = w.contiguous()
        nb = (n + blocksize - 1) // blocksize
        packed = torch.empty(n // 2, dtype=torch.uint8, device=dev)
        absmax = torch.empty(nb, dtype=torch.float32, device=dev)
        rc = N.lib().fmsb_quant4(wc.data_ptr(), n, code.data_ptr(), blocksize, packed.data_ptr(), absmax.data_ptr(),
                                 N.dtype_code(wc.dtype), N.stream_ptr())
        N.check(rc, "fmsb_quant4")
    else:
        packed, absmax = _quant4_ref(w, code, blocksize)
    qs = Quant4State(packed=packed, shape=tuple(w.shape), quant_type=quant_type, blocksize=blocksize, code=code,
                     dtype=dtype or (w.dtype if w.dtype != torch.float32 else torch.bfloat16))
    if not double_quant:
        qs.absmax = absmax
        return qs
    offset = float(absmax.mean().item())
    code2 = dynamic_code_book(dev)
    if w.is_cuda:
        nb = absmax.numel()
        q = torch.empty(nb, dtype=torch.uint8, device=dev)
        absmax2 = torch.empty((nb + 255) // 256, dtype=torch.float32, device=dev)
        rc = N.lib().fmsb_quant8_blockwise(absmax.data_ptr(), nb, offset, code2.data_ptr(), q.data_ptr(),
                                           absmax2.data_ptr(), N.stream_ptr())
        N.check(rc, "fmsb_quant8_blockwise")
    else:
        q, absmax2 = _quant8_ref(absmax, offset, code2)
    qs.absmax_q, qs.code2, qs.absmax2, qs.offset = q, code2, absmax2, offset
    return qs


def dequantize_4bit(qs: Quant4State, dtype: torch.dtype | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    dtype = dtype or qs.dtype
    if not qs.packed.is_cuda:
        dense = dequantize_4bit_ref(qs, dtype)
        if out is None:
            return dense
        out.copy_(dense.view(out.shape))
        return out
    n = qs.numel
    if out is None:
        out = torch.empty(qs.shape, dtype=dtype, device=qs.packed.device)
    code = qs.code if qs.code is not None else code_book(qs.quant_type, qs.packed.device)
    rc = N.lib().fmsb_dequant4(qs.packed.data_ptr(), N.ptr(qs.absmax), N.ptr(qs.absmax_q), N.ptr(qs.code2),
                               N.ptr(qs.absmax2), float(qs.offset), code.data_ptr(), qs.blocksize, n, out.data_ptr(),
                               N.dtype_code(dtype), N.stream_ptr())
    N.check(rc, "fmsb_dequant4")
    return out


# ---------------------------------------------------------------------------------------- GPTQ
def gptq_dequant_ref(qweight, scales, qzeros, g_idx, bits: int, zero_offset: int = 0) -> torch.Tensor:
    """W[in, out] = scales[g_idx] * (unpack(qweight) - (unpack(qzeros)[g_idx] + zero_offset))."""
    per = 32 // bits
    mask = (1 << bits) - 1
    shifts = torch.arange(0, 32, bits, device=qweight.device, dtype=torch.int64)
    qw = (qweight.long() & 0xFFFFFFFF)
    w = ((qw[:, None, :] >> shifts[None, :, None]) & mask).reshape(-1, qweight.shape[1])  # [in, out]
    qz = (qzeros.long() & 0xFFFFFFFF)
    z = ((qz[:, :, None] >> shifts[None, None, :]) & mask).reshape(qzeros.shape[0], -1) + zero_offset  # [G, out]
    g = g_idx.long()
    return (scales[g].float() * (w - z[g]).float()).to(scales.dtype)


def gptq_dequant(qweight, scales, qzeros, g_idx, bits: int, group_size: int, zero_offset: int = 0, out=None):
    """Expand GPTQ packed weights to a dense ``[in, out]`` matrix in the dtype of ``scales``."""
    in_features = qweight.shape[0] * (32 // bits)
    out_features = qweight.shape[1]
    if not qweight.is_cuda:
        if g_idx is None:
            g_idx = torch.arange(in_features, device=qweight.device) // group_size
        dense = gptq_dequant_ref(qweight, scales, qzeros, g_idx, bits, zero_offset)
        if out is None:
            return dense
        out.copy_(dense)
        return out
    if out is None:
        out = torch.empty(in_features, out_features, dtype=scales.dtype, device=qweight.device)
    elif out.shape != (in_features, out_features) or out.stride(1) != 1 or out.dtype != scales.dtype:
        raise ValueError("`out` must be [in, out] with unit column stride and the dtype of the scales")
    rc = N.lib().fmsb_gptq_dequant(qweight.data_ptr(), scales.data_ptr(), qzeros.data_ptr(), N.ptr(g_idx),
                                   in_features, out_features, bits, group_size, zero_offset, out.data_ptr(),
                                   out.stride(0), N.dtype_code(scales.dtype), N.stream_ptr())
    N.check(rc, "fmsb_gptq_dequant")
    return out


def gptq_pack(w_int: torch.Tensor, bits: int) -> torch.Tensor:
    """Pack integer weights ``[in, out]`` (values < 2^bits) along the input rows into int32 ``[in*bits/32, out]``."""
    per = 32 // bits
    i, o = w_int.shape
    v = w_int.long().view(i // per, per, o)
    shifts = torch.arange(0, 32, bits, device=w_int.device, dtype=torch.int64)[None, :, None]
    packed = (v << shifts).sum(dim=1) & 0xFFFFFFFF
    packed = torch.where(packed >= 2 ** 31, packed - 2 ** 32, packed)
    return packed.to(torch.int32)


def gptq_pack_zeros(z_int: torch.Tensor, bits: int) -> torch.Tensor:
    """Pack integer zero points ``[groups, out]`` along the output columns into int32 ``[groups, out*bits/32]``."""
    per = 32 // bits
    g, o = z_int.shape
    v = z_int.long().view(g, o // per, per)
    shifts = torch.arange(0, 32, bits, device=z_int.device, dtype=torch.int64)[None, None, :]
    packed = (v << shifts).sum(dim=2) & 0xFFFFFFFF
    packed = torch.where(packed >= 2 ** 31, packed - 2 ** 32, packed)
    return packed.to(torch.int32)


def gptq_unpack(qweight: torch.Tensor, bits: int) -> torch.Tensor:
    """Inverse of :func:`gptq_pack`: int64 codes ``[in, out]``."""
    shifts = torch.arange(0, 32, bits, device=qweight.device, dtype=torch.int64)
    qw = qweight.long() & 0xFFFFFFFF
    return ((qw[:, None, :] >> shifts[None, :, None]) & ((1 << bits) - 1)).reshape(-1, qweight.shape[1])


def gptq_unpack_zeros(qzeros: torch.Tensor, bits: int) -> torch.Tensor:
    """Inverse of :func:`gptq_pack_zeros`: int64 zero points ``[groups, out]``."""
    shifts = torch.arange(0, 32, bits, device=qzeros.device, dtype=torch.int64)
    qz = qzeros.long() & 0xFFFFFFFF
    return ((qz[:, :, None] >> shifts[None, None, :]) & ((1 << bits) - 1)).reshape(qzeros.shape[0], -1)


# ------------------------------------------------------------------ names the reference's fused-LoRA code uses
def fast_dequantize(W, quant_state: "Quant4State | None" = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """Dense view of a frozen base weight (fms_acceleration_foak/fused_ops/unsloth_lora/utils.py:86-141).

    ``W`` is a ``Linear4bit`` module, or packed 4-bit data with its :class:`Quant4State`, or (no state) an
    already dense tensor, which is returned untouched."""
    if quant_state is None:
        if hasattr(W, "quant_state"):
            return dequantize_4bit(W.quant_state(), out=out)
        return W
    dense = dequantize_4bit(quant_state, out=out)
    # packed data laid out as one row ``[1, n]`` asks for the transposed weight (reference :138-140)
    return dense.t() if isinstance(W, torch.Tensor) and W.dim() == 2 and W.shape[0] == 1 else dense


def fast_gemv(x: torch.Tensor, W, quant_state: "Quant4State | None" = None, out: torch.Tensor | None = None):
    """Inference product of a few rows with a 4-bit weight: ``x [..., in] -> [..., out]``
    (fms_acceleration_foak/fused_ops/unsloth_lora/utils.py:144-206).  The packed weight is streamed once and
    expanded inside the tcgen05 GEMM kernel; nothing dense is written to memory."""
    from .gemm import FUSED_Q4_MAX_ROWS, gemm_q4_fused

    qs = quant_state if quant_state is not None else W.quant_state()
    x2 = x.reshape(-1, x.shape[-1])
    if x2.shape[0] > FUSED_Q4_MAX_ROWS:
        raise ValueError(f"fast_gemv is for at most {FUSED_Q4_MAX_ROWS} rows, got {x2.shape[0]}")
    if x2.stride(1) != 1 or x2.stride(0) % 8:
        x2 = x2.contiguous()
    y = gemm_q4_fused(x2, qs, out=out)
    return y.view(*x.shape[:-1], y.shape[-1])
