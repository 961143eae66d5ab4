"""Uniform affine quantiser for the weight matrices GPTQ works on.

What this framework quantises is always a 2-D slice of a linear weight ``[rows, columns]`` (a whole matrix, or the
columns of one group), with one ``(scale, zero)`` pair per row, so that is the only case implemented: the range of
every row (widened to contain 0) is mapped onto the integer grid ``[0, 2^bits - 1]``, symmetrically around the
middle of the grid when asked to.  The optional clipping search (``mse``) evaluates all shrink factors of the grid at
once instead of looping over them.  Public surface (names of the reference's
fms_acceleration_peft/gptqmodel/quantization/quantizer.py:16-141): ``quantize``, ``Quantizer.configure /
find_params / quantize / enabled / ready`` and the ``scale`` / ``zero`` / ``maxq`` attributes.
"""
from __future__ import annotations

import torch
from torch import nn


def quantize(x: torch.Tensor, scale: torch.Tensor, zero: torch.Tensor, maxq) -> torch.Tensor:
    """``x`` rounded onto the grid and mapped back: ``scale * (clamp(round(x / scale) + zero, 0, maxq) - zero)``."""
    levels = torch.clamp(torch.round(x / scale) + zero, 0, maxq)
    return scale * (levels - zero)


def _row_ranges(w: torch.Tensor, symmetric: bool):
    """Per-row ``(lo, hi)`` containing 0; rows that are entirely zero get ``(-1, 1)`` so their scale is not 0."""
    lo = w.amin(dim=1).clamp(max=0.0)
    hi = w.amax(dim=1).clamp(min=0.0)
    if symmetric:
        bound = torch.maximum(lo.abs(), hi)
        hi = bound
        lo = torch.where(lo < 0, -bound, lo)
    flat = (lo == 0) & (hi == 0)
    return torch.where(flat, torch.full_like(lo, -1.0), lo), torch.where(flat, torch.full_like(hi, 1.0), hi)


class Quantizer(nn.Module):
    """Holds the grid (``maxq``) and, after :meth:`find_params`, one ``scale`` / ``zero`` per row as ``[rows, 1]``."""

    def __init__(self, shape: int = 1):
        super().__init__()
        self.register_buffer("maxq", torch.tensor(0))
        self.register_buffer("scale", torch.zeros(shape))
        self.register_buffer("zero", torch.zeros(shape))
        self.perchannel, self.sym, self.mse = False, True, False
        self.norm, self.grid, self.maxshrink = 2.4, 100, 0.8

    def configure(self, bits: int, perchannel: bool = False, sym: bool = True, mse: bool = False, norm: float = 2.4,
                  grid: int = 100, maxshrink: float = 0.8, **unused):
        """``perchannel``: one pair per row (else one for the whole slice); ``mse``: search the clipping range that
        minimises ``sum |q(w) - w|^norm`` over ``grid * maxshrink`` shrink factors."""
        self.maxq = torch.tensor(2 ** int(bits) - 1)
        self.perchannel, self.sym, self.mse = bool(perchannel), bool(sym), bool(mse)
        self.norm, self.grid, self.maxshrink = float(norm), int(grid), float(maxshrink)

    # ------------------------------------------------------------------
    def _affine(self, lo: torch.Tensor, hi: torch.Tensor):
        scale = (hi - lo) / self.maxq
        if self.sym:
            zero = torch.full_like(scale, float((int(self.maxq) + 1) // 2))
        else:
            zero = torch.round(-lo / scale)
        return scale, zero

    def _clip_search(self, w: torch.Tensor, lo: torch.Tensor, hi: torch.Tensor, scale, zero):
        """All shrink factors at once (in slabs that keep the work tensor below ~256 MB)."""
        steps = int(self.maxshrink * self.grid)
        if steps <= 0:
            return scale, zero
        shrink = 1.0 - torch.arange(steps, device=w.device, dtype=w.dtype) / self.grid      # [S]
        best_err = torch.full((w.shape[0],), float("inf"), device=w.device, dtype=w.dtype)
        slab = max(1, min(steps, (64 << 20) // max(1, w.numel())))
        for s0 in range(0, steps, slab):
            f = shrink[s0: s0 + slab, None]                                                # [s, 1]
            sc = (f * (hi - lo)[None, :]) / self.maxq                                      # [s, rows]
            zp = zero[None, :].expand_as(sc) if self.sym else torch.round(-(f * lo[None, :]) / sc)
            err = (quantize(w[None], sc[..., None], zp[..., None], self.maxq) - w[None]).abs().pow(self.norm).sum(-1)
            e, arg = err.min(dim=0)                                                        # first minimum of the slab
            take = e < best_err
            rows = torch.nonzero(take).flatten()
            best_err = torch.where(take, e, best_err)
            scale = scale.clone()
            zero = zero.clone()
            scale[rows] = sc[arg[rows], rows]
            zero[rows] = zp[arg[rows], rows]
        return scale, zero

    def find_params(self, x: torch.Tensor, weight: bool = True):
        """Set ``scale`` / ``zero`` from the 2-D slice ``x`` ``[rows, columns]`` (``weight=False``: ``x`` holds one
        feature per COLUMN, as activations do, and is transposed first)."""
        if x.dim() != 2:
            raise ValueError("only 2-D slices of linear weights (or 2-D activations) are quantised here")
        w = (x if weight else x.t()).float()
        self.maxq = self.maxq.to(w.device)
        rows = w.shape[0]
        if not self.perchannel:
            w = w.reshape(1, -1)
        lo, hi = _row_ranges(w, self.sym)
        scale, zero = self._affine(lo, hi)
        if self.mse:
            scale, zero = self._clip_search(w, lo, hi, scale, zero)
        if not self.perchannel:
            scale, zero = scale.expand(rows).clone(), zero.expand(rows).clone()
        if weight:
            self.scale, self.zero = scale.reshape(-1, 1), zero.reshape(-1, 1)
        else:
            self.scale, self.zero = scale.reshape(1, -1), zero.reshape(1, -1)

    def quantize(self, x: torch.Tensor) -> torch.Tensor:
        return quantize(x, self.scale, self.zero, self.maxq) if self.ready() else x

    def enabled(self) -> bool:
        return bool(self.maxq > 0)

    def ready(self) -> bool:
        return bool(torch.all(self.scale != 0))
