"""Reusable device scratch buffers.

Kernels launched on one stream run in order, so a scratch buffer (a dequantised weight, a logits chunk)
can be handed out again as soon as the op that used it has been enqueued.  Buffers are keyed by a tag and
grow monotonically; nothing is freed during training, which keeps the caching allocator out of the step.
"""
from __future__ import annotations

import torch

_bufs: dict[tuple, torch.Tensor] = {}


def get(tag: str, numel: int, dtype: torch.dtype, device) -> torch.Tensor:
    dev = torch.device(device)
    key = (tag, dtype, dev.type, dev.index)
    buf = _bufs.get(key)
    if buf is None or buf.numel() < numel:
        buf = torch.empty(numel, dtype=dtype, device=dev)
        _bufs[key] = buf
    return buf[:numel]


def get2d(tag: str, rows: int, cols: int, dtype: torch.dtype, device) -> torch.Tensor:
    return get(tag, rows * cols, dtype, device).view(rows, cols)


def release_all() -> None:
    _bufs.clear()
