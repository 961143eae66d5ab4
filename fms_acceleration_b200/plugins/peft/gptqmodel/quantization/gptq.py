"""The GPTQ layer-wise quantisation algorithm (Frantar et al., 2022).

For a linear layer with weight ``W [out, in]`` and calibration inputs ``X``: accumulate the Hessian proxy
``H = 2/n * sum x x^T``; then walk the input columns in blocks, quantising one column at a time and
pushing the rounding error onto the not-yet-quantised columns with the rows of the upper Cholesky factor of
``H^-1``.  Options: activation ordering (columns sorted by decreasing ``diag(H)``), per-group parameters
(fresh scale / zero every ``group_size`` columns, or pre-computed "static" groups), diagonal damping.
Role of fms_acceleration_peft/gptqmodel/quantization/gptq.py:24-207 in the reference.
"""
from __future__ import annotations

import math
import os
import time
from logging import getLogger

import torch
from torch import nn

from .quantizer import Quantizer

logger = getLogger(__name__)


class GPTQ:
    def __init__(self, layer: nn.Module):
        self.layer = layer
        self.dev = layer.weight.device
        W = self._weight_matrix()
        self.rows, self.columns = W.shape
        self.H = torch.zeros((self.columns, self.columns), device=self.dev, dtype=torch.float32)
        self.nsamples = 0
        self.quantizer = Quantizer()

    def _weight_matrix(self) -> torch.Tensor:
        W = self.layer.weight.data.clone()
        if isinstance(self.layer, nn.Conv2d):
            W = W.flatten(1)
        elif self.layer.__class__.__name__ == "Conv1D":  # transformers' transposed linear
            W = W.t()
        return W.float()

    def add_batch(self, inp: torch.Tensor, out: torch.Tensor = None) -> None:
        """Fold one batch of layer inputs into the running Hessian estimate."""
        if inp.dim() == 2:
            inp = inp.unsqueeze(0)
        batch = inp.shape[0]
        if isinstance(self.layer, nn.Conv2d):
            unfold = nn.Unfold(self.layer.kernel_size, dilation=self.layer.dilation, padding=self.layer.padding,
                               stride=self.layer.stride)
            x = unfold(inp).permute(1, 0, 2).flatten(1)
        else:
            x = inp.reshape(-1, inp.shape[-1]).t()
        total = self.nsamples + batch
        self.H *= self.nsamples / total
        self.nsamples = total
        x = math.sqrt(2.0 / total) * x.float()
        self.H += x @ x.t()

    def fasterquant(self, blocksize: int = 128, percdamp: float = 0.01, group_size: int = -1, actorder: bool = False,
                    static_groups: bool = False):
        """Quantise the layer in place.  Returns ``(scale [out, G], zero [out, G], g_idx [in], duration, avg_loss)``."""
        W = self._weight_matrix()
        tick = time.time()
        if not self.quantizer.ready():
            self.quantizer.find_params(W, weight=True)
        H = self.H
        del self.H
        dead = torch.diag(H) == 0
        H[dead, dead] = 1
        W[:, dead] = 0

        scales, zeros, group_quantizers = [], [], []
        now_idx = 1
        if static_groups and group_size != -1:
            import copy

            for i in range(0, self.columns, group_size):
                q = copy.deepcopy(self.quantizer)
                q.find_params(W[:, i: i + group_size], weight=True)
                scales.append(q.scale)
                zeros.append(q.zero)
                group_quantizers.append(q)

        perm = invperm = None
        if actorder:
            perm = torch.argsort(torch.diag(H), descending=True)
            W = W[:, perm]
            H = H[perm][:, perm]
            invperm = torch.argsort(perm)

        losses = torch.zeros_like(W)
        Qm = torch.zeros_like(W)
        damp = percdamp * torch.mean(torch.diag(H))
        idx = torch.arange(self.columns, device=self.dev)
        H[idx, idx] += damp
        L = torch.linalg.cholesky(H)
        Hinv = torch.linalg.cholesky(torch.cholesky_inverse(L), upper=True)

        for c0 in range(0, self.columns, blocksize):
            c1 = min(c0 + blocksize, self.columns)
            W1 = W[:, c0:c1].clone()
            Q1 = torch.zeros_like(W1)
            E1 = torch.zeros_like(W1)
            L1 = torch.zeros_like(W1)
            Hi = Hinv[c0:c1, c0:c1]
            for j in range(c1 - c0):
                w = W1[:, j]
                d = Hi[j, j]
                if group_size != -1:
                    if not static_groups:
                        if (c0 + j) % group_size == 0:
                            self.quantizer.find_params(W[:, c0 + j: c0 + j + group_size], weight=True)
                        if ((c0 + j) // group_size) - now_idx == -1:
                            scales.append(self.quantizer.scale)
                            zeros.append(self.quantizer.zero)
                            now_idx += 1
                    else:
                        col = c0 + j
                        if actorder:
                            col = int(perm[col])
                        self.quantizer = group_quantizers[col // group_size]
                q = self.quantizer.quantize(w.unsqueeze(1)).flatten()
                Q1[:, j] = q
                L1[:, j] = (w - q) ** 2 / d ** 2
                err = (w - q) / d
                W1[:, j:] -= err.unsqueeze(1) @ Hi[j, j:].unsqueeze(0)
                E1[:, j] = err
            Qm[:, c0:c1] = Q1
            losses[:, c0:c1] = L1 / 2
            W[:, c1:] -= E1 @ Hinv[c0:c1, c1:]

        duration = time.time() - tick
        avg_loss = torch.sum(losses).item() / max(self.nsamples, 1)
        gsz = group_size if group_size != -1 else self.columns
        if static_groups and actorder:
            g_idx = torch.tensor([int(perm[i]) // gsz for i in range(self.columns)], dtype=torch.int32, device=Qm.device)
        else:
            g_idx = torch.tensor([i // gsz for i in range(self.columns)], dtype=torch.int32, device=Qm.device)
        if actorder:
            Qm = Qm[:, invperm]
            g_idx = g_idx[invperm]
        if self.layer.__class__.__name__ == "Conv1D":
            Qm = Qm.t()
        self.layer.weight.data = Qm.reshape(self.layer.weight.shape).to(self.layer.weight.dtype)
        if not scales:
            scales.append(self.quantizer.scale)
            zeros.append(self.quantizer.zero)
        scale = torch.cat(scales, dim=1)
        zero = torch.cat(zeros, dim=1)
        if os.environ.get("DEBUG"):
            logger.debug("gptq layer: %.2fs, avg loss %.6f", duration, avg_loss)
        return scale, zero, g_idx, duration, avg_loss

    def free(self):
        self.H = None
        if torch.cuda.is_available():
            torch.cuda.empty_cache()
