"""Out-parameter building blocks of the ScatterMoE operator (the reference's launchers,
scattermoe_utils/khd/kernels/ops/compileable_ops.py:23-351): expert-ordered gather of rows, per-expert GEMM with
fused gather / scatter of rows and an optional low-rank term, per-expert weight gradient.

They are written over segment-wise matrix products, so they run on any device and serve as the reference statement
of what ``ops/moe.py`` computes with one grouped tensor-core launch per projection (rows placed in 128-row aligned
expert segments by the dispatch kernel, LoRA term accumulated into the same output tile)."""
from __future__ import annotations

from typing import Optional

import torch

from ...custom_op import torch_custom_op

LIBRARY_NAME = "khd"


@torch_custom_op(f"{LIBRARY_NAME}::bincount", mutates_args={})
def compileable_bincount(x: torch.Tensor, minlength: int) -> torch.Tensor:
    return x.bincount(minlength=minlength)


def _segments(sorted_expert_idxs: torch.Tensor, n_experts: int):
    """(expert, first row, end row) of every non-empty expert segment of an expert-sorted list."""
    ends = torch.bincount(sorted_expert_idxs.long(), minlength=n_experts).cumsum(0).tolist()
    start = 0
    for e, end in enumerate(ends):
        if end > start:
            yield e, start, end
        start = end


def scatter2scatter(X: torch.Tensor, W: torch.Tensor, sorted_expert_idxs: torch.Tensor,
                    sorted_scattered_idxs: torch.Tensor, padded_block_idxs: Optional[torch.Tensor], out: torch.Tensor,
                    FAN_OUT: int, x_grouped: bool = False, y_grouped: bool = False, A: Optional[torch.Tensor] = None,
                    B: Optional[torch.Tensor] = None, lora_alp: float = 0.0) -> None:
    """``out`` <- rows times their expert's ``W[e] (+ A[e] B[e] * lora_alp / r)``.  Sorted position ``p`` reads row
    ``p`` of ``X`` (``x_grouped``) or row ``sorted_scattered_idxs[p] // FAN_OUT``, and writes row ``p`` of ``out``
    (``y_grouped``) or row ``sorted_scattered_idxs[p]``.  ``padded_block_idxs`` (the tile schedule of the reference's
    kernel) is not needed."""
    pos = sorted_scattered_idxs.long()
    rows = X if x_grouped else X.index_select(0, pos // FAN_OUT)
    y = out if y_grouped else torch.empty_like(out)
    lora = A is not None and B is not None and lora_alp > 0
    for e, s, t in _segments(sorted_expert_idxs, W.shape[0]):
        acc = rows[s:t] @ W[e]
        if lora:
            acc = acc + ((rows[s:t] @ A[e]) * (lora_alp / A.shape[2])) @ B[e]
        y[s:t] = acc
    if not y_grouped:
        out.index_copy_(0, pos, y)


def group_bwd_W(DY: torch.Tensor, X: torch.Tensor, expert_offsets: torch.Tensor, DW: torch.Tensor, E: int) -> None:
    """``DW[e]`` <- ``X[segment e]^T DY[segment e]`` (zero for an empty segment); ``expert_offsets`` holds where each
    expert's rows end."""
    start = 0
    for e, end in enumerate(expert_offsets.tolist()[:E]):
        if end > start:
            DW[e].copy_(X[start:end].t() @ DY[start:end])
        else:
            DW[e].zero_()
        start = end


def group(A: torch.Tensor, sorted_expert_idxs: torch.Tensor, out: torch.Tensor, coeff: Optional[torch.Tensor] = None,
          fan_out: int = 1) -> None:
    """``out[p]`` <- ``A[idx[p] // fan_out] * coeff[idx[p]]`` where ``idx`` is the expert-ordered list of (token,
    choice) pairs (the argument keeps the reference's name although it holds pair indices, not expert ids)."""
    idx = sorted_expert_idxs.long()
    if A.size(0) * fan_out != idx.numel():
        raise ValueError("the list must name every (row, choice) pair once")
    rows = A.index_select(0, idx // fan_out)
    if coeff is not None:
        rows = rows * coeff.reshape(-1)[idx].to(rows.dtype)[:, None]
    out.copy_(rows)
