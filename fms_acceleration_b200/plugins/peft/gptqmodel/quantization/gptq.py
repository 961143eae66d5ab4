"""Layer-wise GPTQ quantisation (Frantar et al., 2022) of one linear layer.

Given the weight ``W [out, in]`` and calibration inputs, the second-moment matrix ``H = 2/n sum x x^T`` says how much an
error in input column ``j`` matters and how it can be compensated by the columns that come after it.  With ``U`` the upper
Cholesky factor of ``H^-1``, column ``j`` is rounded onto its grid and the residual ``(w_j - q_j) / U_jj`` is subtracted,
weighted by ``U[j, j+1:]``, from the columns still to come.  Columns are processed in blocks so that the bulk of the
update is one matrix product per block.

Organisation here:

* :func:`inverse_cholesky_factor` - dead columns, damping, ``U``;
* :class:`_GroupGrid` - the ``(scale, zero)`` of every column group as two ``[out, groups]`` tensors, filled up front
  (``static_groups``) or when the sweep reaches a group (the weights of a later group have absorbed earlier errors by
  then, so they cannot be known before);
* :func:`_sweep_block` - the sequential part, one block of columns;
* :meth:`GPTQ.fasterquant` - ordering by ``diag(H)`` (``actorder``), the block loop, un-permuting, ``g_idx``.

Public surface as in the reference (fms_acceleration_peft/gptqmodel/quantization/gptq.py:24-207): ``GPTQ(layer)``,
``add_batch``, ``fasterquant`` returning ``(scale, zero, g_idx, seconds, average loss)``, ``free``.
"""
from __future__ import annotations

import math
import time
from logging import getLogger
from typing import Optional

import torch
from torch import nn

from .quantizer import Quantizer, quantize

logger = getLogger(__name__)


def inverse_cholesky_factor(H: torch.Tensor, W: torch.Tensor, percdamp: float) -> torch.Tensor:
    """Upper-triangular ``U`` with ``U^T U = (H + damp I)^-1``.  Input columns that never fired (zero diagonal) are
    taken out of the problem: their weights are set to zero and their diagonal to one.  ``H`` and ``W`` are modified."""
    diag = torch.diagonal(H)
    silent = diag == 0
    diag[silent] = 1.0
    W[:, silent] = 0.0
    diag += percdamp * diag.mean()
    chol = torch.linalg.cholesky(H)
    return torch.linalg.cholesky(torch.cholesky_inverse(chol), upper=True)


class _GroupGrid:
    """Scale and zero point of every (output row, column group)."""

    def __init__(self, template: Quantizer, rows: int, columns: int, group_size: int, device):
        self.template = template
        self.size = group_size if group_size > 0 else columns
        n = -(-columns // self.size)
        self.scale = torch.zeros(rows, n, device=device)
        self.zero = torch.zeros(rows, n, device=device)
        self.known = [False] * n

    def fit(self, g: int, w_slice: torch.Tensor) -> None:
        self.template.find_params(w_slice, weight=True)
        self.scale[:, g] = self.template.scale[:, 0]
        self.zero[:, g] = self.template.zero[:, 0]
        self.known[g] = True

    def fit_all(self, W: torch.Tensor) -> None:
        for g in range(len(self.known)):
            self.fit(g, W[:, g * self.size: (g + 1) * self.size])

    def adopt(self, quantizer: Quantizer) -> None:
        """One group spanning all columns whose parameters the caller has already fitted."""
        self.scale[:, 0] = quantizer.scale[:, 0]
        self.zero[:, 0] = quantizer.zero[:, 0]
        self.known[0] = True


def _sweep_block(Wb: torch.Tensor, Ub: torch.Tensor, groups, grid: _GroupGrid, maxq, refit):
    """Quantise the columns of one block left to right.  ``groups[j]`` is the group of block column ``j``; ``refit(j)``
    is called before a column whose group has no parameters yet.  Returns (quantised block, scaled residuals, loss)."""
    n = Wb.shape[1]
    Qb = torch.empty_like(Wb)
    Eb = torch.empty_like(Wb)
    loss = Wb.new_zeros(())
    for j in range(n):
        g = groups[j]
        if not grid.known[g]:
            refit(j)
        col = Wb[:, j]
        q = quantize(col, grid.scale[:, g], grid.zero[:, g], maxq)
        resid = (col - q) / Ub[j, j]
        Qb[:, j] = q
        Eb[:, j] = resid
        loss = loss + 0.5 * resid.square().sum()
        if j + 1 < n:
            Wb[:, j + 1:] -= torch.outer(resid, Ub[j, j + 1:])
    return Qb, Eb, loss


class GPTQ:
    def __init__(self, layer: nn.Module):
        self.layer = layer
        self.dev = layer.weight.device
        self.transposed = layer.__class__.__name__ == "Conv1D"  # transformers' GPT-2 style linear stores [in, out]
        if not isinstance(layer, nn.Linear) and not self.transposed:
            raise TypeError(f"GPTQ quantises linear layers; got {layer.__class__.__name__}")
        self.rows, self.columns = self._weight().shape
        self.H: Optional[torch.Tensor] = torch.zeros(self.columns, self.columns, device=self.dev)
        self.nsamples = 0
        self.quantizer = Quantizer()

    def _weight(self) -> torch.Tensor:
        w = self.layer.weight.data
        return (w.t() if self.transposed else w).float().clone()

    def add_batch(self, inp: torch.Tensor, out: torch.Tensor = None) -> None:
        """Fold the layer inputs of one calibration batch into ``H`` (a running mean over samples)."""
        n_new = 1 if inp.dim() == 2 else inp.shape[0]
        x = inp.reshape(-1, inp.shape[-1]).float()
        total = self.nsamples + n_new
        self.H.mul_(self.nsamples / total)
        self.H.addmm_(x.t(), x, alpha=2.0 / total)
        self.nsamples = total

    def fasterquant(self, blocksize: int = 128, percdamp: float = 0.01, group_size: int = -1, actorder: bool = False,
                    static_groups: bool = False):
        """Quantise the layer in place.  Returns ``(scale [out, G], zero [out, G], g_idx [in], seconds, avg_loss)``."""
        started = time.time()
        W = self._weight()
        H, self.H = self.H, None
        grouped = group_size != -1
        grid = _GroupGrid(self.quantizer, self.rows, self.columns, group_size, self.dev)
        if not grouped:
            if not self.quantizer.ready():
                self.quantizer.find_params(W, weight=True)
            grid.adopt(self.quantizer)
        U = None
        if grouped and static_groups:
            # parameters from the ORIGINAL weights and the original column order
            silent = torch.diagonal(H) == 0
            W[:, silent] = 0.0
            grid.fit_all(W)
        order = torch.arange(self.columns, device=self.dev)
        if actorder:
            order = torch.argsort(torch.diagonal(H), descending=True)
            W = W[:, order].contiguous()
            H = H[order][:, order].contiguous()
        U = inverse_cholesky_factor(H, W, percdamp)
        # group of every column in processing order: by original position when the groups were fixed up front,
        # by processing position otherwise
        pos = order if (static_groups and grouped) else torch.arange(self.columns, device=self.dev)
        col_group = (pos // grid.size).tolist()

        Q = torch.empty_like(W)
        total_loss = W.new_zeros(())
        for c0 in range(0, self.columns, blocksize):
            c1 = min(c0 + blocksize, self.columns)
            Wb = W[:, c0:c1].clone()

            def refit(j, c0=c0, Wb=Wb):
                # a dynamic group starts at this column; columns of the group inside the block carry the block's pending
                # updates (Wb), those beyond it are current in W
                g = col_group[c0 + j]
                end = min((g + 1) * grid.size, self.columns)
                inside = Wb[:, j: min(j + grid.size, Wb.shape[1])]
                beyond = W[:, c1:end] if end > c1 else W[:, :0]
                grid.fit(g, torch.cat([inside[:, : end - (c0 + j)], beyond], dim=1))

            Qb, Eb, loss = _sweep_block(Wb, U[c0:c1, c0:c1], col_group[c0:c1], grid, self.quantizer.maxq, refit)
            Q[:, c0:c1] = Qb
            total_loss = total_loss + loss
            if c1 < self.columns:
                W[:, c1:].addmm_(Eb, U[c0:c1, c1:], alpha=-1.0)

        g_idx = (pos // grid.size).to(torch.int32)
        if actorder:
            back = torch.argsort(order)
            Q = Q[:, back]
            g_idx = g_idx[back]
        Qw = Q.t() if self.transposed else Q
        self.layer.weight.data = Qw.reshape(self.layer.weight.shape).to(self.layer.weight.dtype)
        seconds = time.time() - started
        avg_loss = float(total_loss) / max(self.nsamples, 1)
        logger.debug("gptq layer: %.2fs, avg loss %.6f", seconds, avg_loss)
        return grid.scale, grid.zero, g_idx, seconds, avg_loss

    def free(self):
        self.H = None
        if torch.cuda.is_available():
            torch.cuda.empty_cache()
