"""Expert-parallel dispatch and combine with library collectives.

``all_to_all_gather_inputs``: every (token, k) pair becomes one row, rows are ordered by global expert, the
per-expert counts are exchanged, then the rows travel with a variable-split all-to-all; the receiver orders what it
got by local expert.  ``scatter_with_routing_weights``: the reverse exchange, then each token sums its k rows scaled
by the routing weights.  Both are differentiable (the backward of an all-to-all is the all-to-all with the splits
swapped).  The split sizes are read on the host, once per call - the synchronisation the fused kernels avoid."""
from __future__ import annotations

from typing import List, Tuple

import torch
import torch.distributed as dist


class _AllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, out_splits: List[int], in_splits: List[int], group):
        ctx.group, ctx.out_splits, ctx.in_splits = group, out_splits, in_splits
        out = x.new_empty((sum(out_splits),) + tuple(x.shape[1:]))
        dist.all_to_all_single(out, x.contiguous(), output_split_sizes=out_splits, input_split_sizes=in_splits, group=group)
        return out

    @staticmethod
    def backward(ctx, grad):
        back = grad.new_empty((sum(ctx.in_splits),) + tuple(grad.shape[1:]))
        dist.all_to_all_single(back, grad.contiguous(), output_split_sizes=ctx.in_splits,
                               input_split_sizes=ctx.out_splits, group=ctx.group)
        return back, None, None, None


def all_to_all_gather_inputs(x: torch.Tensor, top_experts: torch.Tensor, group, top_k: int,
                             experts_per_rank: int) -> Tuple[torch.Tensor, torch.Tensor, dict]:
    """``x [T, H]``, ``top_experts [T, top_k]`` (global expert ids) -> ``(rows [R, H] ordered by local expert,
    local expert id of every row [R], state for the way back)``."""
    world = dist.get_world_size(group)
    E = experts_per_rank * world
    flat = top_experts.reshape(-1).long()
    order = torch.sort(flat, stable=True).indices                       # pairs grouped by global expert
    counts = torch.bincount(flat, minlength=E)                          # [E] rows this rank sends per expert
    recv_counts = torch.empty_like(counts)
    dist.all_to_all_single(recv_counts, counts, group=group)            # [world * experts_per_rank] by sender
    send_splits = counts.view(world, experts_per_rank).sum(1).tolist()  # host synchronisation
    recv_splits = recv_counts.view(world, experts_per_rank).sum(1).tolist()
    rows = x[order // top_k]                                            # a token is replicated top_k times
    got = _AllToAll.apply(rows, recv_splits, send_splits, group)
    # what arrived is ordered (sender, local expert); the experts want (local expert, sender)
    local_of_row = torch.repeat_interleave(
        torch.arange(experts_per_rank, device=x.device).repeat(world), recv_counts.view(-1))
    by_expert = torch.sort(local_of_row, stable=True).indices
    state = {"order": order, "by_expert": by_expert, "send_splits": send_splits, "recv_splits": recv_splits,
             "top_k": top_k, "tokens": x.shape[0], "group": group}
    return got[by_expert], local_of_row[by_expert], state


def scatter_with_routing_weights(y: torch.Tensor, routing_weights: torch.Tensor, state: dict) -> torch.Tensor:
    """``y [R, H]`` (rows in the order :func:`all_to_all_gather_inputs` returned them) -> ``[T, H]``: rows go back
    to their source rank and every token sums its ``top_k`` rows times ``routing_weights [T, top_k]``."""
    undo = torch.empty_like(state["by_expert"])
    undo[state["by_expert"]] = torch.arange(undo.numel(), device=undo.device)
    back = _AllToAll.apply(y[undo], state["send_splits"], state["recv_splits"], state["group"])
    T, k = state["tokens"], state["top_k"]
    pairs = torch.empty_like(back)
    pairs[state["order"]] = back                                        # pair p = token p // k, choice p % k
    return (pairs.view(T, k, -1) * routing_weights.reshape(T, k, 1).to(pairs.dtype)).sum(1)


def no_indices_just_bins(top_expert: torch.Tensor, num_experts: int):
    """``(bins, tokens_per_expert)``: how many (token, k) pairs go to each expert and the inclusive running total,
    i.e. where each expert's rows end once the pairs are sorted by expert (the reference's helper of this name,
    scattermoe_utils/expert_parallel.py:79-92)."""
    tokens_per_expert = torch.bincount(top_expert.reshape(-1).long(), minlength=num_experts).to(torch.int32)
    return tokens_per_expert.cumsum(0).to(torch.int32), tokens_per_expert
