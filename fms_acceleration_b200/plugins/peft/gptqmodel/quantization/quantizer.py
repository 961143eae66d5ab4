"""Uniform affine quantiser used by GPTQ: per-row (or per-group) scale and zero point from the min / max of
the weights, optionally refined by a grid search on the clipping range (the ``mse`` option).
Role of fms_acceleration_peft/gptqmodel/quantization/quantizer.py:16-141 in the reference."""
from __future__ import annotations

import torch
from torch import nn


def quantize(x: torch.Tensor, scale: torch.Tensor, zero: torch.Tensor, maxq) -> torch.Tensor:
    """Round-trip ``x`` through the integer grid ``[0, maxq]``."""
    if maxq < 0:  # ternary special case kept for API compatibility
        return (x > scale / 2).float() * scale + (x < zero / 2).float() * zero
    q = torch.clamp(torch.round(x / scale) + zero, 0, maxq)
    return scale * (q - zero)


class Quantizer(nn.Module):
    def __init__(self, shape: int = 1):
        super().__init__()
        self.register_buffer("maxq", torch.tensor(0))
        self.register_buffer("scale", torch.zeros(shape))
        self.register_buffer("zero", torch.zeros(shape))

    def configure(self, bits: int, perchannel: bool = False, sym: bool = True, mse: bool = False, norm: float = 2.4,
                  grid: int = 100, maxshrink: float = 0.8, trits: bool = False):
        self.maxq = torch.tensor(2 ** bits - 1)
        self.perchannel, self.sym, self.mse = perchannel, sym, mse
        self.norm, self.grid, self.maxshrink = norm, grid, maxshrink
        if trits:
            self.maxq = torch.tensor(-1)

    def find_params(self, x: torch.Tensor, weight: bool = False):
        dev = x.device
        self.maxq = self.maxq.to(dev)
        shape = x.shape
        if self.perchannel:
            if weight:
                x = x.flatten(1)
            else:
                if len(shape) == 4:
                    x = x.permute(1, 0, 2, 3).flatten(1)
                elif len(shape) == 3:
                    x = x.reshape(-1, shape[-1]).t()
                elif len(shape) == 2:
                    x = x.t()
        else:
            x = x.flatten().unsqueeze(0)

        zeros = torch.zeros(x.shape[0], device=dev)
        xmin = torch.minimum(x.min(1).values, zeros)
        xmax = torch.maximum(x.max(1).values, zeros)
        if self.sym:
            xmax = torch.maximum(xmin.abs(), xmax)
            neg = xmin < 0
            xmin = torch.where(neg, -xmax, xmin)
        dead = (xmin == 0) & (xmax == 0)
        xmin = torch.where(dead, -torch.ones_like(xmin), xmin)
        xmax = torch.where(dead, torch.ones_like(xmax), xmax)

        if self.maxq < 0:
            self.scale, self.zero = xmax, xmin
        else:
            self.scale = (xmax - xmin) / self.maxq
            if self.sym:
                self.zero = torch.full_like(self.scale, (self.maxq + 1) / 2)
            else:
                self.zero = torch.round(-xmin / self.scale)

        if self.mse:
            best = torch.full([x.shape[0]], float("inf"), device=dev)
            for i in range(int(self.maxshrink * self.grid)):
                shrink = 1 - i / self.grid
                lo, hi = shrink * xmin, shrink * xmax
                sc = (hi - lo) / self.maxq
                zp = torch.round(-lo / sc) if not self.sym else self.zero
                err = (quantize(x, sc.unsqueeze(1), zp.unsqueeze(1), self.maxq) - x).abs_().pow_(self.norm).sum(1)
                better = err < best
                if torch.any(better):
                    best[better] = err[better]
                    self.scale[better] = sc[better]
                    self.zero[better] = zp[better]

        if not self.perchannel:
            rep = shape[0] if weight else (shape[1] if len(shape) != 3 else shape[2])
            self.scale = self.scale.repeat(rep)
            self.zero = self.zero.repeat(rep)

        if weight:
            view = [-1] + [1] * (len(shape) - 1)
            self.scale = self.scale.reshape(view)
            self.zero = self.zero.reshape(view)
            return
        if len(shape) == 4:
            self.scale, self.zero = self.scale.reshape(1, -1, 1, 1), self.zero.reshape(1, -1, 1, 1)
        elif len(shape) == 3:
            self.scale, self.zero = self.scale.reshape(1, 1, -1), self.zero.reshape(1, 1, -1)
        elif len(shape) == 2:
            self.scale, self.zero = self.scale.unsqueeze(0), self.zero.unsqueeze(0)

    def quantize(self, x):
        return quantize(x, self.scale, self.zero, self.maxq) if self.ready() else x

    def enabled(self):
        return self.maxq > 0

    def ready(self):
        return bool(torch.all(self.scale != 0))
