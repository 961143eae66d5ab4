"""Padding-free causal attention over packed documents (``csrc/attention.cu``).

The reference obtains this from ``flash_attn_varlen_func`` with ``cu_seqlens`` derived from the positions
where ``position_ids == 0`` (fms_acceleration_aadp/flash_attn.py:36-60,108-199).  Here the document
structure is handed to the kernels as per-token ``doc_start`` / ``doc_end`` arrays built from the same
``cu_seqlens``.
"""
from __future__ import annotations

import math
import os

import torch

from .. import _native as N


def doc_bounds_from_cu_seqlens(cu_seqlens: torch.Tensor, total: int | None = None):
    """int32 ``doc_start[t]``, ``doc_end[t]`` for every packed token (device ops only, no host sync when
    ``total`` is given)."""
    cu = cu_seqlens.to(torch.int64)
    if total is None:
        total = int(cu[-1].item())
    pos = torch.arange(total, device=cu.device)
    doc = torch.searchsorted(cu, pos, right=True) - 1
    doc = doc.clamp(min=0, max=cu.numel() - 2)
    return cu[doc].to(torch.int32).contiguous(), cu[doc + 1].to(torch.int32).contiguous()


def cu_seqlens_from_position_ids(position_ids: torch.Tensor) -> torch.Tensor:
    """Document boundaries of a flattened batch: a new document starts wherever the position is 0."""
    flat = position_ids.reshape(-1)
    starts = torch.nonzero(flat == 0, as_tuple=False).reshape(-1)
    end = torch.tensor([flat.numel()], device=flat.device, dtype=starts.dtype)
    return torch.cat([starts, end]).to(torch.int32)


def attention_ref(q, k, v, doc_start, scale=None):
    """fp32 oracle.  q [T, nh, d], k/v [T, nkv, d]."""
    T, nh, d = q.shape
    nkv = k.shape[1]
    scale = scale or 1.0 / math.sqrt(d)
    qf = q.float().transpose(0, 1)
    kf = k.float().repeat_interleave(nh // nkv, dim=1).transpose(0, 1)
    vf = v.float().repeat_interleave(nh // nkv, dim=1).transpose(0, 1)
    s = torch.matmul(qf, kf.transpose(1, 2)) * scale
    idx = torch.arange(T, device=q.device)
    mask = (idx[None, :] <= idx[:, None]) & (idx[None, :] >= doc_start.long()[:, None])
    s = s.masked_fill(~mask[None], float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.matmul(p, vf).transpose(0, 1).contiguous()


# The reference asks flash-attn for a deterministic backward when FLASH_ATTENTION_DETERMINISTIC is set
# (fms_acceleration_aadp/flash_attn.py:152).  Here the variable is accepted and changes nothing: dQ and dK/dV are
# produced by separate kernels that each own their output rows, so no gradient is accumulated with atomics and two
# runs of the same step give the same bits.
DETERMINISTIC_BACKWARD = True


def _fwd(q2, k2, v2, doc_start, doc_end, nh, nkv, d, scale):
    T = q2.shape[0]
    o = torch.empty(T, nh * d, dtype=q2.dtype, device=q2.device)
    lse = torch.empty(nh, T, dtype=torch.float32, device=q2.device)
    st = N.status_word(q2.device)
    rc = N.lib().fmsb_attn_fwd(q2.data_ptr(), q2.stride(0), k2.data_ptr(), k2.stride(0), v2.data_ptr(), v2.stride(0),
                               o.data_ptr(), o.stride(0), lse.data_ptr(), doc_start.data_ptr(), doc_end.data_ptr(),
                               T, nh, nkv, d, float(scale), N.dtype_code(q2.dtype), st.data_ptr(), N.stream_ptr())
    N.check(rc, "fmsb_attn_fwd")
    return o, lse


def _bwd(q2, k2, v2, o, lse, dout, doc_start, doc_end, nh, nkv, d, scale, dq=None, dk=None, dv=None):
    T = q2.shape[0]
    dev = q2.device
    delta = torch.empty(nh, T, dtype=torch.float32, device=dev)
    fmt = N.dtype_code(q2.dtype)
    rc = N.lib().fmsb_attn_delta(o.data_ptr(), dout.data_ptr(), o.stride(0), dout.stride(0), delta.data_ptr(), T, nh,
                                 d, fmt, N.stream_ptr())
    N.check(rc, "fmsb_attn_delta")
    if dq is None:
        dq = torch.empty(T, nh * d, dtype=q2.dtype, device=dev)
    if dk is None:
        dk = torch.empty(T, nkv * d, dtype=q2.dtype, device=dev)
    if dv is None:
        dv = torch.empty(T, nkv * d, dtype=q2.dtype, device=dev)
    st = N.status_word(dev)
    dq_fn, dkv_fn = N.lib().fmsb_attn_bwd_dq3, N.lib().fmsb_attn_bwd_dkv3
    rc = dq_fn(q2.data_ptr(), q2.stride(0), k2.data_ptr(), k2.stride(0), v2.data_ptr(),
                                  v2.stride(0), dout.data_ptr(), dout.stride(0), dq.data_ptr(), dq.stride(0),
                                  lse.data_ptr(), delta.data_ptr(), doc_start.data_ptr(), doc_end.data_ptr(), T, nh,
                                  nkv, d, float(scale), fmt, st.data_ptr(), N.stream_ptr())
    N.check(rc, "fmsb_attn_bwd_dq")
    rc = dkv_fn(q2.data_ptr(), q2.stride(0), k2.data_ptr(), k2.stride(0), v2.data_ptr(),
                v2.stride(0), dout.data_ptr(), dout.stride(0), dk.data_ptr(), dk.stride(0),
                dv.data_ptr(), dv.stride(0), lse.data_ptr(), delta.data_ptr(), doc_start.data_ptr(),
                doc_end.data_ptr(), T, nh, nkv, d, float(scale), fmt, st.data_ptr(),
                N.stream_ptr())
    N.check(rc, "fmsb_attn_bwd_dkv")
    return dq, dk, dv


def _as2d(x):
    T = x.shape[0]
    x2 = x.reshape(T, -1)
    if x2.stride(1) != 1 or x2.stride(0) % 8 != 0:
        x2 = x2.contiguous()
    return x2


class _VarlenAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, doc_start, doc_end, scale):
        T, nh, d = q.shape
        nkv = k.shape[1]
        q2, k2, v2 = _as2d(q), _as2d(k), _as2d(v)
        o, lse = _fwd(q2, k2, v2, doc_start, doc_end, nh, nkv, d, scale)
        ctx.save_for_backward(q2, k2, v2, o, lse, doc_start, doc_end)
        ctx.meta = (nh, nkv, d, scale)
        return o.view(T, nh, d)

    @staticmethod
    def backward(ctx, dout):
        q2, k2, v2, o, lse, doc_start, doc_end = ctx.saved_tensors
        nh, nkv, d, scale = ctx.meta
        T = q2.shape[0]
        dq, dk, dv = _bwd(q2, k2, v2, o, lse, _as2d(dout), doc_start, doc_end, nh, nkv, d, scale)
        return dq.view(T, nh, d), dk.view(T, nkv, d), dv.view(T, nkv, d), None, None, None


def varlen_attention(q, k, v, doc_start, doc_end, scale=None):
    """Causal attention inside each packed document.  q [T, nh, d]; k, v [T, nkv, d]."""
    scale = scale or 1.0 / math.sqrt(q.shape[-1])
    if not q.is_cuda:
        return attention_ref(q, k, v, doc_start, scale).to(q.dtype)
    return _VarlenAttention.apply(q, k, v, doc_start, doc_end, scale)
