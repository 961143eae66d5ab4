"""Row copies between the token layout and the expert-bin layout, as index operations.

The reference runs these as one Triton program per row (scattermoe_utils/megablocks/kernels/gather_scatter.py:37-309);
its expert-parallel baseline needs them only around the library all-to-all.  The training path of this package never
materialises the permutation separately: ``csrc/moe.cu`` writes rows straight into the (peer's) expert buffer and
sums a token's ``top_k`` rows while pulling them back.  These functions state the same copies with ``index_select`` /
``index_copy`` so that code written against the reference's helpers, and the library-collective baseline, keep working
on any device.

Conventions (all as in the reference): ``indices [T * top_k]`` lists the (token, choice) pairs in bin order, pair
``p`` being choice ``p % top_k`` of token ``p // top_k``; ``bin_ids`` is the bin of every listed pair; ``bins`` /
``padded_bins`` are the inclusive running totals of rows (rows + padding) per bin."""
from __future__ import annotations

import torch


def assert_is_tensor(x, ndim):
    if x.ndim != ndim:
        raise ValueError(f"Expected {ndim}-tensor but got {x.ndim}-tensor")


def assert_is_matrix(x):
    assert_is_tensor(x, 2)


def assert_is_vector(x):
    if x.ndim != 1:
        raise ValueError(f"Expected 1-tensor but got {x.ndim}-tensor")


def assert_equal(a, b):
    if a != b:
        raise ValueError(f"Expected dimensions to be equal but got {a} and {b}.")


def _bin_rows(bin_ids: torch.Tensor, bins: torch.Tensor, padded_bins: torch.Tensor) -> torch.Tensor:
    """Row of the bin-ordered buffer that holds listed pair ``i``: its offset inside its bin plus where the bin
    starts once every bin is padded."""
    i = torch.arange(bin_ids.numel(), device=bin_ids.device)
    if padded_bins is bins:
        return i
    b = bin_ids.long()
    start = torch.cat([bins.new_zeros(1), bins[:-1]]).long()
    pstart = torch.cat([padded_bins.new_zeros(1), padded_bins[:-1]]).long()
    return i - start[b] + pstart[b]


def padded_gather(x, indices, bin_ids, weights, bins, padded_bins, top_k):
    """``x [T, H]`` -> ``[padded_bins[-1], H]``: row ``i`` of the bin order is token ``indices[i] // top_k`` (times
    ``weights[indices[i]]`` when given); padding rows are zero."""
    assert_is_matrix(x)
    for v in (indices, bin_ids, bins, padded_bins):
        assert_is_vector(v)
    assert_equal(indices.shape[0], x.shape[0] * top_k)
    assert_equal(bin_ids.shape[0], x.shape[0] * top_k)
    assert_equal(bins.size(), padded_bins.size())
    idx = indices.long()
    rows = x.index_select(0, idx // top_k)
    if weights is not None:
        assert_equal(weights.shape[0], x.shape[0] * top_k)
        rows = (rows.float() * weights.reshape(-1)[idx].float()[:, None]).to(x.dtype)
    if padded_bins is bins:
        return rows
    out = x.new_zeros((int(padded_bins[-1]), x.shape[1]))
    return out.index_copy(0, _bin_rows(bin_ids, bins, padded_bins), rows)


def gather(x, indices, bin_ids, weights, bins, top_k):
    return padded_gather(x, indices, bin_ids, weights, bins, bins, top_k)


def padded_scatter(x, indices, bin_ids, weights, bins, padded_bins, top_k):
    """``x [rows in bin order, H]`` -> ``[T, H]``: listed pair ``i`` takes its row (times ``weights[indices[i]]``)
    and every token sums its ``top_k`` pairs."""
    assert_is_matrix(x)
    for v in (indices, bin_ids, bins, padded_bins):
        assert_is_vector(v)
    assert_equal(indices.shape[0], bin_ids.shape[0])
    assert_equal(bins.size(), padded_bins.size())
    idx = indices.long()
    rows = x if padded_bins is bins else x.index_select(0, _bin_rows(bin_ids, bins, padded_bins))
    if weights is not None:
        assert_equal(indices.shape[0], weights.shape[0])
        rows = (rows.float() * weights.reshape(-1)[idx].float()[:, None]).to(x.dtype)
    tokens = indices.shape[0] // top_k
    pairs = x.new_empty((tokens * top_k, x.shape[1])).index_copy(0, idx, rows)
    return pairs.view(tokens, top_k, -1).sum(dim=1) if top_k > 1 else pairs


def scatter(x, indices, bin_ids, weights, bins, top_k):
    return padded_scatter(x, indices, bin_ids, weights, bins, bins, top_k)


def padded_scatter_wgrad(x, grad, indices, bin_ids, bins, padded_bins, top_k):
    """Gradient of :func:`padded_scatter` with respect to ``weights``: for pair ``p = indices[i]`` the dot product
    of its row of ``x`` with the output gradient of token ``p // top_k``; returned flat, ``[T * top_k]``."""
    assert_is_matrix(x)
    assert_is_matrix(grad)
    for v in (indices, bin_ids, bins, padded_bins):
        assert_is_vector(v)
    assert_equal(indices.shape[0], bin_ids.shape[0])
    assert_equal(bins.size(), padded_bins.size())
    idx = indices.long()
    rows = x if padded_bins is bins else x.index_select(0, _bin_rows(bin_ids, bins, padded_bins))
    dots = (rows.float() * grad.index_select(0, idx // top_k).float()).sum(-1).to(x.dtype)
    return x.new_empty(idx.numel()).index_copy(0, idx, dots)


def scatter_wgrad(x, grad, indices, bin_ids, bins, top_k):
    return padded_scatter_wgrad(x, grad, indices, bin_ids, bins, bins, top_k)
