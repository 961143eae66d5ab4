"""RMSNorm with optional fused residual add (``csrc/elementwise.cu``).

Semantics follow fms_acceleration_foak/kernels/unsloth/rms_layernorm.py:21-128 of the reference:
fp32 statistics, the normalised value rounded to the weight dtype before the multiply, a gemma
variant that scales by ``w + 1`` entirely in fp32.  Unlike the reference the backward can also
produce the weight gradient (needed for full fine-tuning).
"""
from __future__ import annotations

import torch

from .. import _native as N


def rmsnorm_ref(x, w, eps, gemma=False, residual=None):
    """PyTorch oracle.  Returns (y, h) where h = x + residual (or x)."""
    h = x if residual is None else (x.float() + residual.float()).to(x.dtype)
    hf = h.float()
    inv = torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + eps)
    if gemma:
        y = (hf * inv * (w.float() + 1.0)).to(x.dtype)
    else:
        y = ((hf * inv).to(x.dtype).float() * w.float()).to(x.dtype)
    return y, h


def _fwd_native(x2, w, eps, gemma, residual2, want_h):
    rows, H = x2.shape
    y = torch.empty_like(x2)
    h = torch.empty_like(x2) if (residual2 is not None and want_h) else None
    inv = torch.empty(rows, dtype=torch.float32, device=x2.device)
    rc = N.lib().fmsb_rmsnorm_fwd(x2.data_ptr(), N.ptr(residual2), w.data_ptr(), y.data_ptr(), N.ptr(h),
                                  inv.data_ptr(), rows, H, float(eps), int(gemma), N.dtype_code(x2.dtype),
                                  N.stream_ptr())
    N.check(rc, "fmsb_rmsnorm_fwd")
    return y, h, inv


def _bwd_native(dy2, h2, w, inv, gemma, dres2, need_dw):
    rows, H = h2.shape
    dx = torch.empty_like(h2)
    dw = partial = None
    nblk = 0
    if need_dw:
        nblk = min(rows, 148 * (4 if H <= 2048 else 2))  # CTAs of the launch, one partial row of dw each
        partial = torch.empty(nblk, H, dtype=torch.float32, device=h2.device)
        dw = torch.empty(H, dtype=torch.float32, device=h2.device)
    rc = N.lib().fmsb_rmsnorm_bwd(dy2.data_ptr(), h2.data_ptr(), w.data_ptr(), inv.data_ptr(), N.ptr(dres2),
                                  dx.data_ptr(), N.ptr(partial), N.ptr(dw), nblk, rows, H, int(gemma),
                                  N.dtype_code(h2.dtype), N.stream_ptr())
    N.check(rc, "fmsb_rmsnorm_bwd")
    return dx, dw


class _RMSNorm(torch.autograd.Function):
    """y = norm(x); also usable with a fused residual: (y, h) = norm(x + r), x + r."""

    @staticmethod
    def forward(ctx, x, w, eps, gemma, residual):
        shape = x.shape
        x2 = x.reshape(-1, shape[-1]).contiguous()
        r2 = None if residual is None else residual.reshape(-1, shape[-1]).contiguous()
        y, h, inv = _fwd_native(x2, w.contiguous(), eps, gemma, r2, True)
        hsave = h if h is not None else x2
        ctx.save_for_backward(hsave, w, inv)
        ctx.gemma = gemma
        ctx.has_res = residual is not None
        ctx.shape = shape
        if residual is None:
            return y.view(shape)
        return y.view(shape), h.view(shape)

    @staticmethod
    def backward(ctx, dy, dh=None):
        h2, w, inv = ctx.saved_tensors
        dy2 = dy.reshape(h2.shape).contiguous()
        dres = None if dh is None else dh.reshape(h2.shape).contiguous()
        dx, dw = _bwd_native(dy2, h2, w, inv, ctx.gemma, dres, ctx.needs_input_grad[1])
        dx = dx.view(ctx.shape)
        dwo = None if dw is None else dw.to(w.dtype)
        return dx, dwo, None, None, (dx if ctx.has_res else None)


def rmsnorm(x, w, eps=1e-6, gemma=False, residual=None):
    """RMSNorm.  With ``residual`` returns ``(norm(x + residual), x + residual)``."""
    if not x.is_cuda:
        y, h = rmsnorm_ref(x, w, eps, gemma, residual)
        return y if residual is None else (y, h)
    return _RMSNorm.apply(x, w, eps, gemma, residual)


def fast_rms_layernorm(layernorm, X, gemma: bool = False):
    """Module-level entry used by the patch rules (same role as ``fast_rms_layernorm`` in the
    reference, fms_acceleration_foak/kernels/unsloth/rms_layernorm.py:187-192)."""
    eps = getattr(layernorm, "variance_epsilon", None)
    if eps is None:
        eps = getattr(layernorm, "eps", 1e-6)
    return rmsnorm(X, layernorm.weight, eps, gemma)
