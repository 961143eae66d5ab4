"""Python front-end of the tcgen05 GEMM (``csrc/gemm_tcgen05.cu``).

``gemm(a, b)`` computes ``alpha * (op(a) @ op(b)^T + op(a2) @ op(b2)^T) + beta * c`` with fp32
accumulation in tensor memory.  Operand orientation is described by two flags instead of
transposed copies:

* ``a_mn=False``: ``a`` is ``[M, K]`` (contraction contiguous); ``a_mn=True``: ``a`` is ``[K, M]``.
* ``b_mn=False``: ``b`` is ``[N, K]`` (an ``nn.Linear`` weight); ``b_mn=True``: ``b`` is ``[K, N]``.

So ``y = x W^T`` is ``gemm(x, W)``, ``dx = dy W`` is ``gemm(dy, W, b_mn=True)`` and
``dW = dy^T x`` is ``gemm(dy, x, a_mn=True, b_mn=True)``.
"""
from __future__ import annotations

import torch

import ctypes as _ct

from .. import _native as N
from .. import _native as _NV  # second alias: `N` is also the name of a matrix dimension argument below

N.declare("fmsb_batched_gemm", [_ct.c_void_p, _ct.c_longlong, _ct.c_longlong, _ct.c_longlong, _ct.c_void_p, _ct.c_longlong,
                                 _ct.c_longlong, _ct.c_longlong, _ct.c_int, _ct.c_int, _ct.c_int, _ct.c_void_p, _ct.c_longlong,
                                 _ct.c_int, _ct.c_void_p, _ct.c_longlong, _ct.c_float, _ct.c_float, _ct.c_int, _ct.c_int,
                                 _ct.c_int, _ct.c_int, _ct.c_void_p, _ct.c_void_p, _ct.c_void_p])


def _pick_bn(n: int, b_mn: bool) -> int:
    if n >= 192:
        bn = 256
    elif n > 64:
        bn = 128
    elif n > 32:
        bn = 64
    elif n > 16:
        bn = 32
    else:
        bn = 16
    if b_mn and bn < 64:
        bn = 64
    return bn


def _check_operand(t: torch.Tensor, name: str) -> None:
    if t.dim() != 2:
        raise ValueError(f"{name} must be 2-D")
    if t.stride(1) != 1:
        raise ValueError(f"{name} must have unit stride in its last dimension")
    if t.stride(0) % 8 != 0 or t.data_ptr() % 16 != 0:
        raise ValueError(f"{name}: leading dimension must be a multiple of 8 elements and 16-byte aligned")


def _gemm_host(a, b, a_mn, b_mn, a2, b2, c, alpha, beta, out, out_dtype):
    """The contract of :func:`gemm` stated with torch operators for tensors that live on the host (any floating
    dtype, fp32 accumulation): ``out = alpha * (op(a) op(b) + op(a2) op(b2)) + beta * c`` with ``op(a) = a^T`` when
    ``a_mn`` and ``op(b) = b`` when ``b_mn`` (else ``b^T``).  What the CPU tests of the layers above run on; a tensor
    on a GPU never comes here."""
    def prod(x, y):
        x = (x.t() if a_mn else x).float()
        y = (y if b_mn else y.t()).float()
        return x @ y

    acc = prod(a, b)
    if a2 is not None:
        acc = acc + prod(a2, b2)
    acc = acc * alpha
    if c is not None and beta != 0.0:
        acc = acc + beta * c.float()
    if out is None:
        return acc.to(out_dtype or a.dtype)
    out.copy_(acc)
    return out


def gemm(
    a: torch.Tensor,
    b: torch.Tensor,
    *,
    a_mn: bool = False,
    b_mn: bool = False,
    a2: torch.Tensor | None = None,
    b2: torch.Tensor | None = None,
    c: torch.Tensor | None = None,
    alpha: float = 1.0,
    beta: float = 0.0,
    out: torch.Tensor | None = None,
    out_dtype: torch.dtype | None = None,
    bn: int | None = None,
    max_ctas: int = 0,
) -> torch.Tensor:
    if not a.is_cuda:
        return _gemm_host(a, b, a_mn, b_mn, a2, b2, c, alpha, beta, out, out_dtype)
    if a.dtype not in (torch.bfloat16, torch.float16) or b.dtype != a.dtype:
        raise TypeError("gemm operands must both be bf16 or both fp16")
    _check_operand(a, "a")
    _check_operand(b, "b")
    M, K = (a.shape[1], a.shape[0]) if a_mn else (a.shape[0], a.shape[1])
    Nn, Kb = (b.shape[1], b.shape[0]) if b_mn else (b.shape[0], b.shape[1])
    if K != Kb:
        raise ValueError(f"contraction mismatch: {K} vs {Kb}")
    K2 = 0
    if a2 is not None:
        _check_operand(a2, "a2")
        _check_operand(b2, "b2")
        M2, K2 = (a2.shape[1], a2.shape[0]) if a_mn else (a2.shape[0], a2.shape[1])
        N2, K2b = (b2.shape[1], b2.shape[0]) if b_mn else (b2.shape[0], b2.shape[1])
        if (M2, N2) != (M, Nn) or K2 != K2b:
            raise ValueError("second operand pair has mismatching shape")
    if out is None:
        out = torch.empty(M, Nn, dtype=out_dtype or a.dtype, device=a.device)
    else:
        if out.shape != (M, Nn) or out.stride(1) != 1:
            raise ValueError("bad `out`")
    if out.dtype not in (a.dtype, torch.float32):
        raise TypeError("output must have the operand dtype or fp32")
    if c is not None:
        if c.shape != (M, Nn) or c.stride(1) != 1 or c.dtype != a.dtype:
            raise ValueError("bad `c`")
    if bn is None:
        bn = _pick_bn(Nn, b_mn)
    if a_mn and b_mn and a2 is None and c is None and alpha == 1.0 and max_ctas == 0:
        splits = _split_k(M, Nn, K, bn)
        if splits > 1:
            return _gemm_split_k(a, b, M, Nn, K, splits, out, bn)
    status = N.status_word(a.device)
    rc = N.lib().fmsb_gemm(
        a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0), K,
        N.ptr(a2), a2.stride(0) if a2 is not None else 0, N.ptr(b2), b2.stride(0) if b2 is not None else 0, K2,
        int(a_mn), int(b_mn),
        out.data_ptr(), out.stride(0), int(out.dtype == torch.float32),
        N.ptr(c), c.stride(0) if c is not None else 0,
        float(alpha), float(beta), M, Nn, N.dtype_code(a.dtype), bn, int(max_ctas),
        status.data_ptr(), N.stream_ptr(),
    )
    N.check(rc, "fmsb_gemm")
    return out


def set_pair_mode(mode: int) -> int:
    """Choose between the single-CTA tile kernel and the CTA-pair kernel (256 x 256 tiles, ``cta_group::2``) for plain
    products: 0 never, 1 when the product has enough tiles to fill the machine (default), 2 whenever M, N >= 256.
    Returns the previous setting."""
    N.declare("fmsb_gemm_set_pair_mode", [_ct.c_int])
    return int(N.lib().fmsb_gemm_set_pair_mode(int(mode)))


def set_pair_store(tma_store: int) -> int:
    """Epilogue of the CTA-pair kernel for 16-bit outputs: 1 (default) stages the tile through shared memory and
    stores it with bulk tensor stores, 0 uses per-thread 16-byte stores.  Returns the previous setting."""
    N.declare("fmsb_gemm_set_pair_store", [_ct.c_int])
    return int(N.lib().fmsb_gemm_set_pair_store(int(tma_store)))


SM_COUNT = 148
SPLIT_K_MIN = 512  # shortest contraction slice worth a tile of its own


def _split_k(M: int, Nn: int, K: int, bn: int) -> int:
    """Number of contraction slices for a weight-gradient product (``a^T b`` with a long contraction, the token
    axis): when the output has fewer tiles than half the SMs, the contraction is cut so that every SM gets a tile."""
    tiles = -(-M // 128) * -(-Nn // bn)
    if tiles * 2 > SM_COUNT or K < 2 * SPLIT_K_MIN:
        return 1
    splits = 1
    while tiles * splits * 2 <= 2 * SM_COUNT and K % (splits * 2 * 64) == 0 and K // (splits * 2) >= SPLIT_K_MIN:
        splits *= 2
    return splits


def _gemm_split_k(a, b, M, Nn, K, splits, out, bn):
    """``a [K, M]^T b [K, N]`` as ``splits`` batched products over slices of the contraction, partial results in
    fp32, then one sum."""
    part = torch.empty(splits * M, Nn, dtype=torch.float32, device=a.device)
    ks = K // splits
    batched_gemm(a, b, M=M, N=Nn, K=ks, n_batch=splits, n_inner=1, a_off=(ks, 0, 0, 1), b_off=(ks, 0, 0, 1),
                 d_off=(M, 0, 0), a_mn=True, b_mn=True, out=part, bn=bn)
    if out.dtype == torch.float32:
        return torch.sum(part.view(splits, M, Nn), dim=0, out=out)
    out.copy_(part.view(splits, M, Nn).sum(0))
    return out


def linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``x @ w.T`` for ``x [..., K]`` and ``w [N, K]``."""
    lead = x.shape[:-1]
    y = gemm(x.reshape(-1, x.shape[-1]), w)
    return y.reshape(*lead, w.shape[0])


def batched_gemm(a, b, *, M, N, K, n_batch, n_inner=1, a_off=(0, 0, 0, 1), b_off=(0, 0, 0, 1), d_off=(0, 0, 0),
                 a_mn=False, b_mn=False, out=None, out_rows=None, out_cols=None, out_dtype=None, bn=None):
    """Uniform batched GEMM over windows of stored 2-D matrices (``fmsb_batched_gemm``).

    Batch index ``(o, i)`` with ``i < n_inner``; ``x_off = (row step per o, row step per i, column step per i,
    divisor applied to i for the column step)`` addresses the STORED matrix (for an MN-major operand its rows are the
    contraction index); ``d_off = (row step per o, row step per i, column step per i)``.
    """
    import ctypes

    if out is None:
        out = torch.empty(out_rows, out_cols, dtype=out_dtype or a.dtype, device=a.device)
    if bn is None:
        bn = _pick_bn(N, b_mn)
    desc = (ctypes.c_int * 13)(n_batch, n_inner, a_off[0], a_off[1], a_off[2], a_off[3], b_off[0], b_off[1], b_off[2],
                               b_off[3], d_off[0], d_off[1], d_off[2])
    st = _NV.status_word(a.device)
    rc = _NV.lib().fmsb_batched_gemm(a.data_ptr(), a.stride(0), a.shape[0], a.shape[1], b.data_ptr(), b.stride(0),
                                    b.shape[0], b.shape[1], K, int(a_mn), int(b_mn), out.data_ptr(), out.stride(0),
                                    int(out.dtype == torch.float32), None, 0, 1.0, 0.0, M, N, _NV.dtype_code(a.dtype), bn,
                                    desc, st.data_ptr(), _NV.stream_ptr())
    _NV.check(rc, "fmsb_batched_gemm")
    return out


# ------------------------------------------------------------------------------------------------
# fused gather + 4-bit dequantise + GEMM + LoRA for few rows (csrc/gemm_q4_fused.cu)
# ------------------------------------------------------------------------------------------------
N.declare("fmsb_gemm_q4_fused", [_ct.c_void_p, _ct.c_longlong, _ct.c_void_p, _ct.c_longlong, _ct.c_int, _ct.c_void_p,
                                  _ct.c_void_p, _ct.c_void_p, _ct.c_void_p, _ct.c_float, _ct.c_void_p, _ct.c_void_p,
                                  _ct.c_longlong, _ct.c_void_p, _ct.c_longlong, _ct.c_int, _ct.c_void_p, _ct.c_longlong,
                                  _ct.c_float, _ct.c_int, _ct.c_int, _ct.c_int, _ct.c_int, _ct.c_int, _ct.c_void_p,
                                  _ct.c_void_p])

_CODE16_HOST: dict = {}


def _code16_host(quant_type: str):
    arr = _CODE16_HOST.get(quant_type)
    if arr is None:
        from .quant import FP4_CODE, NF4_CODE

        vals = {"nf4": NF4_CODE, "fp4": FP4_CODE}[quant_type]
        arr = (_ct.c_float * 16)(*[float(v) for v in vals])
        _CODE16_HOST[quant_type] = arr
    return arr


FUSED_Q4_MAX_ROWS = 128  # above this the weight is dequantised once and the plain GEMM is used


def gemm_q4_fused(x: torch.Tensor, qs, xa: torch.Tensor | None = None, bl: torch.Tensor | None = None,
                  shard_ptrs=None, shard_bytes: int | None = None, alpha: float = 1.0, out: torch.Tensor | None = None,
                  bn: int | None = None) -> torch.Tensor:
    """``x [M, K] @ dequant(qs) [N, K]^T (+ xa [M, R] @ bl [N, R]^T)`` without materialising the 16-bit weight.

    ``qs`` is a ``Quant4State`` of a ``[N, K]`` weight with block size 64.  ``shard_ptrs`` (a ctypes array of
    ``world`` device pointers, each ``shard_bytes`` long) replaces ``qs.packed`` when the flat packed array lives in
    equal shards on several GPUs; the kernel then reads the peers' shards directly.
    """
    if qs.blocksize != 64:
        raise ValueError("the fused kernel needs quantisation blocks of 64 values")
    Nn, K = qs.shape
    M = x.shape[0]
    if x.dtype not in (torch.bfloat16, torch.float16) or x.stride(1) != 1 or x.stride(0) % 8 or K % 64 or Nn % 8:
        raise ValueError("x must be a 16-bit row-major matrix; K % 64 == 0 and N % 8 == 0")
    if out is None:
        out = torch.empty(M, Nn, dtype=x.dtype, device=x.device)
    if shard_ptrs is None:
        world, shard_bytes = 1, (qs.packed.numel() + 31) // 32 * 32
        shard_ptrs = (_ct.c_void_p * 1)(qs.packed.data_ptr())
    else:
        world = len(shard_ptrs)
    if bn is None:
        # enough CTAs to put every SM to work on a thin problem
        bn = 128 if (Nn // 128) * ((M + 127) // 128) >= 148 else (64 if (Nn // 64) * ((M + 127) // 128) >= 148 else 32)
    code_host = _code16_host(qs.quant_type)  # host constants: no device read on the launch path
    r2 = 0
    if xa is not None:
        if bl is None or xa.shape[0] != M or bl.shape[0] != Nn or xa.shape[1] != bl.shape[1]:
            raise ValueError("LoRA pair: xa [M, R] and bl [N, R]")
        r2 = xa.shape[1]
    st = N.status_word(x.device)
    rc = N.lib().fmsb_gemm_q4_fused(
        x.data_ptr(), x.stride(0), shard_ptrs, int(shard_bytes), world, N.ptr(qs.absmax), N.ptr(qs.absmax_q),
        N.ptr(qs.code2), N.ptr(qs.absmax2), float(qs.offset), code_host, N.ptr(xa), xa.stride(0) if xa is not None else 0,
        N.ptr(bl), bl.stride(0) if bl is not None else 0, r2, out.data_ptr(), out.stride(0), float(alpha), M, Nn, K,
        N.dtype_code(x.dtype), bn, st.data_ptr(), N.stream_ptr())
    N.check(rc, "fmsb_gemm_q4_fused")
    return out


N.declare("fmsb_gemm_gptq_fused", [_ct.c_void_p, _ct.c_longlong, _ct.c_void_p, _ct.c_void_p, _ct.c_void_p, _ct.c_int,
                                    _ct.c_int, _ct.c_void_p, _ct.c_longlong, _ct.c_void_p, _ct.c_longlong, _ct.c_int,
                                    _ct.c_void_p, _ct.c_longlong, _ct.c_float, _ct.c_int, _ct.c_int, _ct.c_int,
                                    _ct.c_int, _ct.c_int, _ct.c_void_p, _ct.c_void_p])


def gemm_gptq_fused(x: torch.Tensor, qweight: torch.Tensor, scales: torch.Tensor, qzeros: torch.Tensor,
                    group_size: int, zero_offset: int = 0, xa: torch.Tensor | None = None,
                    bl: torch.Tensor | None = None, alpha: float = 1.0, out: torch.Tensor | None = None,
                    bn: int | None = None) -> torch.Tensor:
    """``x [M, K] @ W [K, N] (+ xa [M, R] @ bl [N, R]^T)`` for a GPTQ int4 weight, dequantised inside the GEMM.

    ``qweight [K/8, N]`` int32, ``scales [K/group, N]`` in the dtype of ``x``, ``qzeros [K/group, N/8]`` int32; groups
    in input-feature order (no activation reordering), ``group_size % 64 == 0``.  The few-row counterpart of the
    reference's fused Triton kernels (gptqmodel/nn_modules/triton_utils/kernels.py:105-201); with many rows the
    weight is dequantised once (``ops.quant.gptq_dequant``) and the plain GEMM runs.
    """
    K, Nn = qweight.shape[0] * 8, qweight.shape[1]
    M = x.shape[0]
    if x.dtype not in (torch.bfloat16, torch.float16) or x.stride(1) != 1 or x.stride(0) % 8 or K % 64 or Nn % 8:
        raise ValueError("x must be a 16-bit row-major matrix; K % 64 == 0 and N % 8 == 0")
    if group_size % 64 or K % group_size or scales.dtype != x.dtype or not (
            qweight.is_contiguous() and scales.is_contiguous() and qzeros.is_contiguous()):
        raise ValueError("group_size % 64 == 0, scales in the dtype of x, contiguous packed tensors")
    if out is None:
        out = torch.empty(M, Nn, dtype=x.dtype, device=x.device)
    if bn is None:
        bn = 128 if (Nn // 128) * ((M + 127) // 128) >= 148 else (64 if (Nn // 64) * ((M + 127) // 128) >= 148 else 32)
    r2 = 0
    if xa is not None:
        if bl is None or xa.shape[0] != M or bl.shape[0] != Nn or xa.shape[1] != bl.shape[1]:
            raise ValueError("LoRA pair: xa [M, R] and bl [N, R]")
        r2 = xa.shape[1]
    st = N.status_word(x.device)
    rc = N.lib().fmsb_gemm_gptq_fused(
        x.data_ptr(), x.stride(0), qweight.data_ptr(), scales.data_ptr(), qzeros.data_ptr(), int(group_size),
        int(zero_offset), N.ptr(xa), xa.stride(0) if xa is not None else 0, N.ptr(bl),
        bl.stride(0) if bl is not None else 0, r2, out.data_ptr(), out.stride(0), float(alpha), M, Nn, K,
        N.dtype_code(x.dtype), bn, st.data_ptr(), N.stream_ptr())
    N.check(rc, "fmsb_gemm_gptq_fused")
    return out
