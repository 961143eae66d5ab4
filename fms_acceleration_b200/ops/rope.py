"""Rotary position embedding with explicit position ids (``csrc/elementwise.cu``).

The reference kernel (fms_acceleration_foak/kernels/unsloth/rope_embedding.py:20-72) rotates the two
halves of each head and recovers the position as ``row % seqlen``; that is wrong for packed,
padding-free batches, so this op always takes the position of every token.
"""
from __future__ import annotations

import torch

from .. import _native as N


def rope_tables(head_dim: int, max_pos: int, theta: float, device) -> tuple[torch.Tensor, torch.Tensor]:
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device=device) / head_dim))
    ang = torch.arange(max_pos, dtype=torch.float32, device=device)[:, None] * inv_freq[None, :]
    return ang.cos().contiguous(), ang.sin().contiguous()


def rope_ref(x, pos, cos_t, sin_t, sign=1.0):
    """x: [T, n_heads, d]; pos: [T]; tables [max_pos, d/2]."""
    d = x.shape[-1]
    c = cos_t[pos.long()][:, None, :].float()
    s = sin_t[pos.long()][:, None, :].float() * sign
    x1, x2 = x[..., : d // 2].float(), x[..., d // 2:].float()
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).to(x.dtype)


def rope_inplace_(buf: torch.Tensor, n_heads: int, head_dim: int, pos: torch.Tensor, cos_t, sin_t, sign=1.0):
    """Rotate the first ``n_heads`` heads of every row of the packed 2-D buffer ``buf`` in place."""
    assert buf.dim() == 2 and buf.stride(1) == 1
    if not buf.is_cuda:
        T = buf.shape[0]
        v = buf[:, : n_heads * head_dim].reshape(T, n_heads, head_dim)
        buf[:, : n_heads * head_dim] = rope_ref(v, pos, cos_t, sin_t, sign).reshape(T, -1)
        return buf
    pos32 = pos if pos.dtype == torch.int32 else pos.to(torch.int32)
    rc = N.lib().fmsb_rope(buf.data_ptr(), pos32.data_ptr(), cos_t.data_ptr(), sin_t.data_ptr(), buf.shape[0],
                           n_heads, head_dim, buf.stride(0), float(sign), N.dtype_code(buf.dtype), N.stream_ptr())
    N.check(rc, "fmsb_rope")
    return buf


class _Rope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, pos, cos_t, sin_t):
        # x: [T, n_heads, d]
        T, nh, d = x.shape
        out = x.contiguous().clone().view(T, nh * d)
        rope_inplace_(out, nh, d, pos, cos_t, sin_t, 1.0)
        ctx.save_for_backward(pos, cos_t, sin_t)
        return out.view(T, nh, d)

    @staticmethod
    def backward(ctx, dy):
        pos, cos_t, sin_t = ctx.saved_tensors
        T, nh, d = dy.shape
        g = dy.contiguous().clone().view(T, nh * d)
        rope_inplace_(g, nh, d, pos, cos_t, sin_t, -1.0)
        return g.view(T, nh, d), None, None, None


def apply_rope(x, pos, cos_t, sin_t):
    """x: [T, n_heads, d] -> rotated copy (differentiable)."""
    if not x.is_cuda:
        return rope_ref(x, pos, cos_t, sin_t)
    return _Rope.apply(x, pos, cos_t, sin_t)


def fast_rope_embedding(q, k, cos, sin, position_ids=None, unsqueeze_dim=1):
    """HF-shaped entry: q,k ``[B, heads, S, d]``, cos/sin ``[B, S, d]`` (already gathered per token).
    Mirrors fms_acceleration_foak/kernels/unsloth/rope_embedding.py:136-139 but honours positions."""
    B, Hq, S, d = q.shape
    half = d // 2
    if cos.dim() == 2:  # [S, d]
        cos, sin = cos[None], sin[None]
    if cos.shape[0] != B:  # one set of positions broadcast over the batch
        cos, sin = cos.expand(B, S, d), sin.expand(B, S, d)
    cos_t = cos.reshape(B * S, d)[:, :half].float().contiguous()
    sin_t = sin.reshape(B * S, d)[:, :half].float().contiguous()
    pos = torch.arange(B * S, device=q.device, dtype=torch.int32)

    def run(x):
        Hx = x.shape[1]
        xt = x.transpose(1, 2).reshape(B * S, Hx, d)
        return apply_rope(xt, pos, cos_t, sin_t).view(B, S, Hx, d).transpose(1, 2)

    return run(q), run(k)
