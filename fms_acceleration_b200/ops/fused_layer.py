"""Whole-block fused forward/backward for a pre-norm decoder layer on packed tokens.

One autograd node per block instead of one per op: the attention block is
``x + W_o . attention(rope(W_qkv . rmsnorm(x)))`` and the MLP block is
``h + W_down . glu(W_gate_up . rmsnorm(h))``, each projection being a :class:`ProjGroup` (dense / NF4 / GPTQ
base weight, optional LoRA).  The residual adds ride in the GEMM epilogues, the q/k rotation and the gated
activation run in place on the GEMM outputs, and only what the backward needs is kept.

Covers what the reference assembles from per-module patches: fused LoRA QKV / O / MLP
(fms_acceleration_foak/models/utils.py:60-224, fused_ops/unsloth_lora/*/fast_lora.py), fast RMSNorm and RoPE
(kernels/unsloth/rms_layernorm.py, rope_embedding.py) and varlen flash attention
(fms_acceleration_aadp/flash_attn.py:108-199).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional

import torch

from . import activation as ACT
from . import attention as ATT
from . import rmsnorm as RN
from .proj import ProjGroup
from .rope import rope_inplace_


@dataclass
class PackedBatch:
    """Token-packed batch: every tensor is indexed by the flattened token position."""

    pos: torch.Tensor        # int32 [T] position inside its document
    doc_start: torch.Tensor  # int32 [T]
    doc_end: torch.Tensor    # int32 [T]
    cos: torch.Tensor        # fp32 [max_pos, d/2]
    sin: torch.Tensor

    @classmethod
    def from_position_ids(cls, position_ids: torch.Tensor, cos, sin) -> "PackedBatch":
        flat = position_ids.reshape(-1)
        cu = ATT.cu_seqlens_from_position_ids(flat)
        ds, de = ATT.doc_bounds_from_cu_seqlens(cu, flat.numel())
        return cls(flat.to(torch.int32).contiguous(), ds, de, cos, sin)

    @classmethod
    def from_cu_seqlens(cls, cu_seqlens: torch.Tensor, total: int, cos, sin) -> "PackedBatch":
        ds, de = ATT.doc_bounds_from_cu_seqlens(cu_seqlens, total)
        pos = (torch.arange(total, device=ds.device, dtype=torch.int32) - ds).contiguous()
        return cls(pos, ds, de, cos, sin)


def _norm_eps(norm) -> float:
    eps = getattr(norm, "variance_epsilon", None)
    return float(eps if eps is not None else getattr(norm, "eps", 1e-6))


class AttentionBlockSpec:
    """Static description of one attention block (built once per layer)."""

    def __init__(self, norm, q_proj, k_proj, v_proj, o_proj, n_heads, n_kv_heads, head_dim, tag,
                 softmax_scale: Optional[float] = None, residual_multiplier: float = 1.0, gemma_norm: bool = False):
        self.norm = norm
        self.qkv = ProjGroup([q_proj, k_proj, v_proj], tag + ".qkv")
        self.o = ProjGroup([o_proj], tag + ".o")
        self.nh, self.nkv, self.d = n_heads, n_kv_heads, head_dim
        self.scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(head_dim)
        self.res_mult = residual_multiplier
        self.gemma = gemma_norm

    def trainable(self) -> List[torch.Tensor]:
        t = []
        if self.norm.weight.requires_grad:
            t.append(self.norm.weight)
        return t + self.qkv.trainable() + self.o.trainable()


class MLPBlockSpec:
    def __init__(self, norm, gate_proj, up_proj, down_proj, act: str, tag, residual_multiplier: float = 1.0,
                 gemma_norm: bool = False):
        self.norm = norm
        self.gate_up = ProjGroup([gate_proj, up_proj], tag + ".gate_up")
        self.down = ProjGroup([down_proj], tag + ".down")
        self.inter = self.gate_up.out_sizes[0]
        self.act = act
        self.res_mult = residual_multiplier
        self.gemma = gemma_norm

    def trainable(self) -> List[torch.Tensor]:
        t = []
        if self.norm.weight.requires_grad:
            t.append(self.norm.weight)
        return t + self.gate_up.trainable() + self.down.trainable()


def _scaled(t: torch.Tensor, m: float) -> torch.Tensor:
    return t if m == 1.0 else t * m


class _AttentionBlock(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, spec: AttentionBlockSpec, batch: PackedBatch, *params):
        T, H = x.shape
        nh, nkv, d = spec.nh, spec.nkv, spec.d
        y1, _, inv1 = RN._fwd_native(x, spec.norm.weight, _norm_eps(spec.norm), spec.gemma, None, False)
        ctx.aux_qkv, ctx.aux_o = {}, {}
        qkv, xa_qkv = spec.qkv.forward(y1, aux=ctx.aux_qkv)
        rope_inplace_(qkv, nh + nkv, d, batch.pos, batch.cos, batch.sin, 1.0)
        q2 = qkv[:, : nh * d]
        k2 = qkv[:, nh * d: (nh + nkv) * d]
        v2 = qkv[:, (nh + nkv) * d:]
        o_attn, lse = ATT._fwd(q2, k2, v2, batch.doc_start, batch.doc_end, nh, nkv, d, spec.scale)
        if spec.res_mult == 1.0:
            h, xa_o = spec.o.forward(o_attn, residual=x, aux=ctx.aux_o)
        else:
            part, xa_o = spec.o.forward(o_attn, aux=ctx.aux_o)
            h = torch.add(x, part, alpha=spec.res_mult)
        ctx.spec, ctx.batch = spec, batch
        ctx.save_for_backward(x, inv1, y1, qkv, o_attn, lse, xa_qkv, xa_o)
        return h

    @staticmethod
    def backward(ctx, dh):
        spec, batch = ctx.spec, ctx.batch
        x, inv1, y1, qkv, o_attn, lse, xa_qkv, xa_o = ctx.saved_tensors
        nh, nkv, d = spec.nh, spec.nkv, spec.d
        dh = dh.contiguous()
        d_oattn, g_o = spec.o.backward(_scaled(dh, spec.res_mult), o_attn, xa_o, aux=ctx.aux_o)
        dqkv = torch.empty_like(qkv)
        q2 = qkv[:, : nh * d]
        k2 = qkv[:, nh * d: (nh + nkv) * d]
        v2 = qkv[:, (nh + nkv) * d:]
        ATT._bwd(q2, k2, v2, o_attn, lse, d_oattn, batch.doc_start, batch.doc_end, nh, nkv, d, spec.scale,
                 dq=dqkv[:, : nh * d], dk=dqkv[:, nh * d: (nh + nkv) * d], dv=dqkv[:, (nh + nkv) * d:])
        rope_inplace_(dqkv, nh + nkv, d, batch.pos, batch.cos, batch.sin, -1.0)
        need_dx = ctx.needs_input_grad[0]
        norm_trains = spec.norm.weight.requires_grad
        dy1, g_qkv = spec.qkv.backward(dqkv, y1, xa_qkv, need_dx=need_dx or norm_trains, aux=ctx.aux_qkv)
        dx = None
        grads: List[Optional[torch.Tensor]] = []
        if need_dx or norm_trains:
            dx, dw = RN._bwd_native(dy1, x, spec.norm.weight, inv1, spec.gemma, dh, norm_trains)
            if norm_trains:
                grads.append(dw.to(spec.norm.weight.dtype))
        grads += g_qkv + g_o
        return (dx, None, None, *grads)


class _MLPBlock(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h, spec: MLPBlockSpec, *params):
        I = spec.inter
        y2, _, inv2 = RN._fwd_native(h, spec.norm.weight, _norm_eps(spec.norm), spec.gemma, None, False)
        ctx.aux_gu, ctx.aux_d = {}, {}
        gu, xa_gu = spec.gate_up.forward(y2, aux=ctx.aux_gu)
        act = ACT.glu_fwd(gu[:, :I], gu[:, I:], spec.act)
        if spec.res_mult == 1.0:
            out, xa_d = spec.down.forward(act, residual=h, aux=ctx.aux_d)
        else:
            part, xa_d = spec.down.forward(act, aux=ctx.aux_d)
            out = torch.add(h, part, alpha=spec.res_mult)
        keep_y2 = len(spec.gate_up.trainable()) > 0
        ctx.spec = spec
        ctx.keep_y2 = keep_y2
        ctx.save_for_backward(h, inv2, gu, y2 if keep_y2 else None, xa_gu, xa_d)
        return out

    @staticmethod
    def backward(ctx, dout):
        spec = ctx.spec
        h, inv2, gu, y2, xa_gu, xa_d = ctx.saved_tensors
        I = spec.inter
        dout = dout.contiguous()
        act = None
        if len(spec.down.trainable()) > 0:
            act = ACT.glu_fwd(gu[:, :I], gu[:, I:], spec.act)
        dact, g_d = spec.down.backward(_scaled(dout, spec.res_mult), act, xa_d, aux=ctx.aux_d)
        # in place: gu <- (d gate | d up)
        ACT.glu_bwd(dact, gu[:, :I], gu[:, I:], spec.act, de=gu[:, :I], dg=gu[:, I:])
        if y2 is None and len(spec.gate_up.trainable()) > 0:
            y2, _, _ = RN._fwd_native(h, spec.norm.weight, _norm_eps(spec.norm), spec.gemma, None, False)
        dy2, g_gu = spec.gate_up.backward(gu, y2, xa_gu, aux=ctx.aux_gu)
        norm_trains = spec.norm.weight.requires_grad
        dh, dw = RN._bwd_native(dy2, h, spec.norm.weight, inv2, spec.gemma, dout, norm_trains)
        grads: List[Optional[torch.Tensor]] = []
        if norm_trains:
            grads.append(dw.to(spec.norm.weight.dtype))
        grads += g_gu + g_d
        return (dh, None, *grads)


def attention_block(x: torch.Tensor, spec: AttentionBlockSpec, batch: PackedBatch) -> torch.Tensor:
    return _AttentionBlock.apply(x, spec, batch, *spec.trainable())


def mlp_block(h: torch.Tensor, spec: MLPBlockSpec) -> torch.Tensor:
    return _MLPBlock.apply(h, spec, *spec.trainable())
