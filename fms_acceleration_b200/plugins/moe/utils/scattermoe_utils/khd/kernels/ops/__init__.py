"""``scattered_experts``: one expert projection of a mixture-of-experts layer over rows that stay in token order
(gathered into expert order on the way in, scattered back on the way out), differentiable, with an optional
per-expert LoRA pair and an optional gate-weighted sum over a token's ``k`` rows.  Same contract as the reference's
operator (scattermoe_utils/khd/kernels/ops/__init__.py:26-310).

``ScatterMoE.forward`` of this package does not come through here: it hands the whole gated MLP (both projections,
activation, combine) to ``ops/moe.py``, which keeps rows in 128-row aligned expert segments between the two grouped
GEMMs instead of scattering and re-gathering them.  This operator exists for code that drives ``ScatteredExperts``
modules directly."""
from __future__ import annotations

import torch

from .compileable_ops import compileable_bincount, group, group_bwd_W, scatter2scatter  # noqa: F401

BLOCK_M = 128


def padded_block_indices(sorted_experts_idxs: torch.Tensor, k: int, N_BLOCK_SIZE: int = BLOCK_M):
    """``(first row of every N_BLOCK_SIZE-row tile when each expert's rows start a new tile, where each expert's rows
    end)`` for an expert-sorted list over ``k`` experts."""
    counts = sorted_experts_idxs.bincount(minlength=k)
    ends = counts.cumsum(-1)
    tiles = (counts + N_BLOCK_SIZE - 1) // N_BLOCK_SIZE
    expert_of_tile = torch.repeat_interleave(torch.arange(k, device=counts.device), tiles)
    first_tile = tiles.cumsum(-1) - tiles
    within = torch.arange(expert_of_tile.numel(), device=counts.device) - first_tile[expert_of_tile]
    starts = (ends - counts)[expert_of_tile] + within * N_BLOCK_SIZE
    return starts.to(sorted_experts_idxs.dtype), ends


class _ScatteredExperts(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, expert_weights, k, sorted_expert_idxs, sorted_scattered_idxs, padded_block_idxs, expert_offsets,
                gates=None, grouped_in=False, grouped_out=False, expert_lora_A=None, expert_lora_B=None,
                lora_alp: float = 0.0):
        rows = x.new_empty(sorted_expert_idxs.size(0), expert_weights.size(-1))
        scatter2scatter(x, expert_weights, sorted_expert_idxs, sorted_scattered_idxs, padded_block_idxs, rows, k,
                        grouped_in, grouped_out, expert_lora_A, expert_lora_B, lora_alp)
        ctx.lora = lora_alp > 0 and expert_lora_A is not None and expert_lora_B is not None
        ctx.lora_alp = lora_alp
        per_token = None
        out = rows
        if gates is not None:
            per_token = rows.view(gates.size(0), gates.size(1), rows.size(-1))
            out = torch.bmm(gates.unsqueeze(1), per_token).squeeze(1)
        ctx.save_for_backward(x, expert_weights, sorted_expert_idxs, sorted_scattered_idxs, expert_offsets, gates,
                              per_token, *((expert_lora_A, expert_lora_B) if ctx.lora else ()))
        ctx.k, ctx.grouped_in, ctx.grouped_out = k, grouped_in, grouped_out
        return out

    @staticmethod
    def backward(ctx, grad_out):
        x, W, sorted_expert_idxs, sorted_scattered_idxs, expert_offsets, gates, per_token, *ab = ctx.saved_tensors
        k = ctx.k
        grad_out = grad_out.contiguous()
        d_gates = None
        fan, coeff = 1, None
        if gates is not None:
            d_gates = torch.bmm(per_token, grad_out.unsqueeze(2)).squeeze(-1)
            fan, coeff = gates.size(1), gates.flatten()
        # output gradient and input rows in expert order
        if ctx.grouped_out:
            dy = grad_out
        else:
            dy = grad_out.new_empty(grad_out.shape[0] * fan, grad_out.shape[1])
            group(grad_out, sorted_scattered_idxs, dy, coeff=coeff, fan_out=fan)
        if ctx.grouped_in:
            xs = x
        else:
            xs = x.new_empty(sorted_scattered_idxs.size(0), x.size(1))
            group(x, sorted_scattered_idxs, xs, fan_out=k)
        dW = dy.new_empty(W.shape)
        group_bwd_W(dy, xs, expert_offsets, dW, W.size(0))
        dA = dB = None
        extra = {}
        if ctx.lora:
            A, B = ab
            s = ctx.lora_alp / A.size(-1)
            dA = dW @ B.transpose(1, 2) * s
            dB = A.transpose(1, 2) @ dW * s
            dW = None
            extra = {"A": B.transpose(1, 2), "B": A.transpose(1, 2), "lora_alp": ctx.lora_alp}
        elif not ctx.needs_input_grad[1]:
            dW = None
        d_rows = x.new_empty(sorted_expert_idxs.size(0), W.size(1))
        scatter2scatter(dy, W.transpose(1, 2), sorted_expert_idxs, sorted_scattered_idxs, None, d_rows, 1, True,
                        ctx.grouped_in, **extra)
        dx = d_rows if k == 1 else d_rows.view(x.size(0), k, d_rows.size(-1)).sum(-2)
        return dx, dW, None, None, None, None, None, d_gates, None, None, dA, dB, None


def scattered_experts(inputs, expert_weights, k, sorted_expert_idxs, sorted_scattered_idxs, padded_block_idxs,
                      expert_offsets, gates=None, grouped_in=False, grouped_out=False, expert_lora_A=None,
                      expert_lora_B=None, lora_alp: float = 0.0):
    return _ScatteredExperts.apply(inputs, expert_weights, k, sorted_expert_idxs, sorted_scattered_idxs,
                                   padded_block_idxs, expert_offsets, gates, grouped_in, grouped_out, expert_lora_A,
                                   expert_lora_B, lora_alp)
