"""Differentiable forms of the row permutations and of the variable-split all-to-all, under the names the reference
vendors (scattermoe_utils/megablocks/autograd.py:17-183).

Three facts carry the whole file: the gradient of a gather is the scatter over the same index lists, the gradient of a
scatter is the gather (plus, for the routing weights, one dot product per (token, choice) pair), and the gradient of
an all-to-all is the all-to-all with the two split lists exchanged.  ``custom_fwd`` / ``custom_bwd`` make the
functions behave under autocast: the forward runs once in the autocast dtype with autocast switched off inside, the
backward with autocast off."""
from __future__ import annotations

import functools

import torch
import torch.distributed as dist

from .kernels import gather_scatter as _rows


# ----------------------------------------------------------------------------------------------------- autocast
def _is_eligible(x) -> bool:
    return torch.is_tensor(x) and x.is_cuda and x.is_floating_point() and x.dtype is not torch.float64


def _cast(x, dtype):
    """``x`` with every eligible tensor inside it (lists, tuples, dicts) converted to ``dtype``."""
    if _is_eligible(x):
        return x.to(dtype)
    if isinstance(x, dict):
        return {k: _cast(v, dtype) for k, v in x.items()}
    if isinstance(x, (list, tuple)):
        return type(x)(_cast(v, dtype) for v in x)
    return x


def _outside_autocast(fn, cast_arguments: bool):
    @functools.wraps(fn)
    def run(*args, **kwargs):
        if cast_arguments and not torch.is_autocast_enabled():
            return fn(*args, **kwargs)
        if cast_arguments:
            low = torch.get_autocast_dtype("cuda")
            args, kwargs = _cast(args, low), _cast(kwargs, low)
        with torch.autocast(device_type="cuda", enabled=False):
            return fn(*args, **kwargs)

    return run


def custom_fwd(fwd):
    return _outside_autocast(fwd, cast_arguments=True)


def custom_bwd(bwd):
    return _outside_autocast(bwd, cast_arguments=False)


# ----------------------------------------------------------------------------------------------------- all-to-all
class AllToAllOp(torch.autograd.Function):
    """``apply(x, output_split_sizes, input_split_sizes, group, async_op) -> (rows received, handle)``."""

    @staticmethod
    def forward(ctx, x, output_split_sizes, input_split_sizes, group, async_op):
        ctx.sent_shape, ctx.group = x.shape, group
        ctx.splits = (list(output_split_sizes), list(input_split_sizes))
        received = x.new_empty((sum(output_split_sizes),) + tuple(x.shape[1:]))
        handle = dist.all_to_all_single(received, x.contiguous(), output_split_sizes=ctx.splits[0],
                                        input_split_sizes=ctx.splits[1], group=group, async_op=async_op)
        return received, handle

    @staticmethod
    def backward(ctx, grad, _handle_grad):
        if not ctx.needs_input_grad[0]:
            return (None,) * 5
        came_back = grad.new_empty(ctx.sent_shape)
        got, sent = ctx.splits
        dist.all_to_all_single(came_back, grad.contiguous(), output_split_sizes=sent, input_split_sizes=got,
                               group=ctx.group)
        return (came_back,) + (None,) * 4


def all_to_all(x, output_split_sizes, input_split_sizes, group, async_op=False):
    """The handle is None unless ``async_op``."""
    return AllToAllOp.apply(x, output_split_sizes, input_split_sizes, group, async_op)


# ------------------------------------------------------------------------------------------------ gather / scatter
class GatherOp(torch.autograd.Function):
    """Token rows -> bin order (every token ``top_k`` times)."""

    @staticmethod
    @custom_fwd
    def forward(ctx, x, indices, bin_ids, bins, top_k):
        ctx.top_k = top_k
        ctx.save_for_backward(indices, bin_ids, bins)
        return _rows.gather(x, indices, bin_ids, None, bins, top_k)

    @staticmethod
    @custom_bwd
    def backward(ctx, grad):
        indices, bin_ids, bins = ctx.saved_tensors
        return (_rows.scatter(grad.contiguous(), indices, bin_ids, None, bins, ctx.top_k),) + (None,) * 4


class ScatterOp(torch.autograd.Function):
    """Bin order -> token rows, each token summing its ``top_k`` rows times ``weights`` (None: plain sum)."""

    @staticmethod
    @custom_fwd
    def forward(ctx, x, indices, bin_ids, weights, bins, top_k):
        ctx.top_k = top_k
        ctx.weighted = weights is not None and ctx.needs_input_grad[3]
        ctx.save_for_backward(indices, bin_ids, weights, bins, *([x] if ctx.weighted else []))
        return _rows.scatter(x, indices, bin_ids, weights, bins, top_k)

    @staticmethod
    @custom_bwd
    def backward(ctx, grad):
        indices, bin_ids, weights, bins, *kept = ctx.saved_tensors
        grad = grad.contiguous()
        d_rows = d_weights = None
        if ctx.needs_input_grad[0]:
            d_rows = _rows.gather(grad, indices, bin_ids, weights, bins, ctx.top_k)
        if ctx.weighted:
            d_weights = _rows.scatter_wgrad(kept[0], grad, indices, bin_ids, bins, ctx.top_k).reshape(weights.shape)
        return d_rows, None, None, d_weights, None, None


gather = GatherOp.apply
scatter = ScatterOp.apply
