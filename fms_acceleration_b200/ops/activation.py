"""Gated activations: SwiGLU, GEGLU (exact and tanh approximation) (``csrc/elementwise.cu``).

Reference: fms_acceleration_foak/fused_ops/unsloth_lora/swiglu.py:20-98 and geglu.py:20-202.
``h = act(e) * g``; the backward produces ``de`` and ``dg`` (the reference writes them in place
over ``e`` and ``g``; here in place is optional).
"""
from __future__ import annotations


import torch
import torch.nn.functional as F

from .. import _native as N

ACT_CODES = {"silu": 0, "swiglu": 0, "gelu": 1, "gelu_exact": 1, "gelu_pytorch_tanh": 2, "gelu_tanh": 2, "gelu_new": 2}


def glu_ref(e, g, act="silu"):
    code = ACT_CODES[act]
    ef = e.float()
    if code == 0:
        f = F.silu(ef)
    elif code == 1:
        f = F.gelu(ef)
    else:
        f = F.gelu(ef, approximate="tanh")
    return (f.to(e.dtype).float() * g.float()).to(e.dtype)


def glu_fwd(e, g, act="silu", out=None, rows_dev=None):
    """e, g: 2-D views (row stride arbitrary, unit column stride) -> h [rows, I].  ``rows_dev``: optional int32
    device scalar with the number of rows in use (the rest of a fixed-capacity buffer is left untouched)."""
    rows, I = e.shape
    if out is None:
        out = torch.empty(rows, I, dtype=e.dtype, device=e.device)
    rc = N.lib().fmsb_glu_fwd(e.data_ptr(), g.data_ptr(), out.data_ptr(), rows, I, e.stride(0), g.stride(0),
                              out.stride(0), ACT_CODES[act], N.dtype_code(e.dtype), N.ptr(rows_dev), N.stream_ptr())
    N.check(rc, "fmsb_glu_fwd")
    return out


def glu_bwd(dh, e, g, act="silu", de=None, dg=None, h_out=None, rows_dev=None):
    rows, I = e.shape
    if de is None:
        de = torch.empty(rows, I, dtype=e.dtype, device=e.device)
    if dg is None:
        dg = torch.empty(rows, I, dtype=e.dtype, device=e.device)
    rc = N.lib().fmsb_glu_bwd(dh.data_ptr(), e.data_ptr(), g.data_ptr(), de.data_ptr(), dg.data_ptr(), N.ptr(h_out),
                              rows, I, dh.stride(0), e.stride(0), g.stride(0), de.stride(0), dg.stride(0),
                              h_out.stride(0) if h_out is not None else 0, ACT_CODES[act], N.dtype_code(e.dtype),
                              N.ptr(rows_dev), N.stream_ptr())
    N.check(rc, "fmsb_glu_bwd")
    return de, dg


class _GLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, e, g, act):
        e2 = e.reshape(-1, e.shape[-1])
        g2 = g.reshape(-1, g.shape[-1])
        if e2.stride(1) != 1:
            e2 = e2.contiguous()
        if g2.stride(1) != 1:
            g2 = g2.contiguous()
        h = glu_fwd(e2, g2, act)
        ctx.save_for_backward(e2, g2)
        ctx.act = act
        ctx.shape = e.shape
        return h.view(e.shape)

    @staticmethod
    def backward(ctx, dh):
        e2, g2 = ctx.saved_tensors
        dh2 = dh.reshape(e2.shape)
        if dh2.stride(1) != 1:
            dh2 = dh2.contiguous()
        de, dg = glu_bwd(dh2, e2, g2, ctx.act)
        return de.view(ctx.shape), dg.view(ctx.shape), None


def glu(e, g, act="silu"):
    if not e.is_cuda:
        return glu_ref(e, g, act)
    return _GLU.apply(e, g, act)


def swiglu_fg_kernel(e, g):
    return glu(e, g, "silu")


def geglu_exact_forward_kernel(e, g):
    return glu(e, g, "gelu")


def geglu_approx_forward_kernel(e, g):
    return glu(e, g, "gelu_pytorch_tanh")
