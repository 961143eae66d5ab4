"""Differentiable forms of the row permutations and of the variable-split all-to-all (the reference's
scattermoe_utils/megablocks/autograd.py:17-183): the backward of a gather is the scatter over the same indices and
the other way round, the backward of an all-to-all is the all-to-all with the split lists swapped."""
from __future__ import annotations

import functools

import torch
import torch.distributed as dist

from .kernels.gather_scatter import gather as _gather
from .kernels.gather_scatter import scatter as _scatter
from .kernels.gather_scatter import scatter_wgrad as _scatter_wgrad


def _is_eligible(x):
    return isinstance(x, torch.Tensor) and x.is_floating_point() and x.is_cuda and x.dtype is not torch.float64


def _cast(x, dtype):
    if isinstance(x, torch.Tensor) and _is_eligible(x):
        return x.to(dtype)
    if isinstance(x, dict):
        return {_cast(k, dtype): _cast(v, dtype) for k, v in x.items()}
    if isinstance(x, (list, tuple)):
        return type(x)(_cast(v, dtype) for v in x)
    return x


def custom_fwd(fwd):
    """Run ``forward`` in the autocast dtype (arguments cast once, autocast off inside) when autocast is on."""

    @functools.wraps(fwd)
    def decorate(*args, **kwargs):
        if torch.is_autocast_enabled():
            dtype = torch.get_autocast_dtype("cuda")
            with torch.autocast(device_type="cuda", enabled=False):
                return fwd(*_cast(args, dtype), **_cast(kwargs, dtype))
        return fwd(*args, **kwargs)

    return decorate


def custom_bwd(bwd):
    """Run ``backward`` with autocast off: the gradients already carry the dtype the forward chose."""

    @functools.wraps(bwd)
    def decorate(*args, **kwargs):
        with torch.autocast(device_type="cuda", enabled=False):
            return bwd(*args, **kwargs)

    return decorate


class AllToAllOp(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, output_split_sizes, input_split_sizes, group, async_op):
        out = x.new_empty((sum(output_split_sizes),) + tuple(x.shape[1:]))
        ctx.input_shape = x.shape
        ctx.output_split_sizes, ctx.input_split_sizes, ctx.group = output_split_sizes, input_split_sizes, group
        handle = dist.all_to_all_single(out, x.contiguous(), output_split_sizes=output_split_sizes,
                                        input_split_sizes=input_split_sizes, group=group, async_op=async_op)
        return out, handle

    @staticmethod
    def backward(ctx, grad, _):
        if not ctx.needs_input_grad[0]:
            return None, None, None, None, None
        back = grad.new_empty(ctx.input_shape)
        dist.all_to_all_single(back, grad.contiguous(), output_split_sizes=ctx.input_split_sizes,
                               input_split_sizes=ctx.output_split_sizes, group=ctx.group)
        return back, None, None, None, None


def all_to_all(x, output_split_sizes, input_split_sizes, group, async_op=False):
    """``(received rows, handle)``; the handle is None unless ``async_op``."""
    return AllToAllOp.apply(x, output_split_sizes, input_split_sizes, group, async_op)


class ScatterOp(torch.autograd.Function):
    @staticmethod
    @custom_fwd
    def forward(ctx, x, indices, bin_ids, weights, bins, top_k):
        keep_x = [x] if ctx.needs_input_grad[3] else []
        ctx.save_for_backward(indices, bin_ids, weights, bins, *keep_x)
        ctx.top_k = top_k
        return _scatter(x, indices, bin_ids, weights, bins, top_k)

    @staticmethod
    @custom_bwd
    def backward(ctx, grad):
        grad = grad.contiguous()
        indices, bin_ids, weights, bins = ctx.saved_tensors[:4]
        dx = _gather(grad, indices, bin_ids, weights, bins, ctx.top_k) if ctx.needs_input_grad[0] else None
        dw = None
        if ctx.needs_input_grad[3]:
            dw = _scatter_wgrad(ctx.saved_tensors[-1], grad, indices, bin_ids, bins, ctx.top_k).reshape(weights.shape)
        return dx, None, None, dw, None, None


def scatter(x, indices, bin_ids, weights, bins, top_k):
    return ScatterOp.apply(x, indices, bin_ids, weights, bins, top_k)


class GatherOp(torch.autograd.Function):
    @staticmethod
    @custom_fwd
    def forward(ctx, x, indices, bin_ids, bins, top_k):
        ctx.save_for_backward(indices, bin_ids, bins)
        ctx.top_k = top_k
        return _gather(x, indices, bin_ids, None, bins, top_k)

    @staticmethod
    @custom_bwd
    def backward(ctx, grad):
        indices, bin_ids, bins = ctx.saved_tensors
        return _scatter(grad.contiguous(), indices, bin_ids, None, bins, ctx.top_k), None, None, None, None


gather = GatherOp.apply
