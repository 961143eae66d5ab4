"""Projection groups: one or more linear projections that read the same input and whose outputs are laid out
side by side (q|k|v, gate|up) or a single projection (o, down), each optionally carrying a LoRA adapter and
each with a dense, 4-bit (NF4/FP4) or GPTQ base weight.

This is the B200 counterpart of the reference's fused LoRA autograd functions
(fms_acceleration_foak/fused_ops/unsloth_lora/bnb/fast_lora.py:21-471 and gptq/fast_lora.py:174-859):
``y = x W^T + s (x A^T) B^T`` per projection, backward with analytic ``dA``/``dB`` and ``dx`` through a
freshly dequantised ``W``.  Differences in mechanism: the projections of a group run as ONE tcgen05 GEMM over
the concatenated weight, and the LoRA update is accumulated in the same tensor-memory accumulator through the
GEMM's second operand pair (A2 = s * x A_cat^T, B2 = block-diagonal lora_B), so the output is written once.
"""
from __future__ import annotations

from typing import List, Optional

import torch
from torch import nn

from . import workspace as WS
from .gemm import gemm


def _unwrap(mod: nn.Module):
    """(base_module, lora_module_or_None)"""
    if hasattr(mod, "base_layer") and hasattr(mod, "lora_A"):
        return mod.base_layer, mod
    return mod, None


def _lora_parts(lora_mod):
    name = lora_mod.active_adapters[0] if hasattr(lora_mod, "active_adapters") else "default"
    if isinstance(name, (list, tuple)):
        name = name[0]
    A = lora_mod.lora_A[name].weight
    B = lora_mod.lora_B[name].weight
    s = lora_mod.scaling[name]
    return A, B, float(s)


class ProjGroup:
    def __init__(self, mods: List[nn.Module], tag: str):
        self.tag = tag
        self.bases, self.loras = [], []
        for m in mods:
            b, l = _unwrap(m)
            self.bases.append(b)
            self.loras.append(l)
        self.out_sizes = [self._out(b) for b in self.bases]
        self.in_features = self._in(self.bases[0])
        self.total_out = sum(self.out_sizes)
        self.offsets = [0]
        for o in self.out_sizes:
            self.offsets.append(self.offsets[-1] + o)
        self.has_lora = any(l is not None for l in self.loras)
        self.kind = self._kind(self.bases[0])

    @staticmethod
    def _out(b):
        return getattr(b, "out_features", None) or b.outfeatures

    @staticmethod
    def _in(b):
        return getattr(b, "in_features", None) or b.infeatures

    @staticmethod
    def _kind(b):
        n = b.__class__.__name__
        if n == "Linear4bit":
            return "q4"
        if hasattr(b, "qweight"):
            return "gptq"
        return "dense"

    # ------------------------------------------------------------------ parameters that receive gradients
    def trainable(self) -> List[torch.Tensor]:
        out = []
        for b, l in zip(self.bases, self.loras):
            if self.kind == "dense" and b.weight.requires_grad:
                out.append(b.weight)
            if l is not None:
                A, B, _ = _lora_parts(l)
                out += [A, B]
        return out

    # ------------------------------------------------------------------ base weight as one dense matrix
    def dense_weight(self, dtype, device):
        """Returns (W, b_mn).  b_mn=False: W is [total_out, in]; b_mn=True (GPTQ): W is [in, total_out]."""
        if self.kind == "dense":
            if len(self.bases) == 1:
                return self.bases[0].weight, False
            W = WS.get2d("wcat_" + self.tag, self.total_out, self.in_features, dtype, device)
            for b, o0, o1 in zip(self.bases, self.offsets[:-1], self.offsets[1:]):
                W[o0:o1].copy_(b.weight)
            return W, False
        if self.kind == "q4":
            W = WS.get2d("wdeq", self.total_out, self.in_features, dtype, device)
            for b, o0, o1 in zip(self.bases, self.offsets[:-1], self.offsets[1:]):
                b.dequantize(out=W[o0:o1], dtype=dtype)
            return W, False
        # gptq: dequantised layout is [in, out]; concatenate along columns
        W = WS.get2d("wdeq", self.in_features, self.total_out, dtype, device)
        if len(self.bases) == 1:
            self.bases[0].dequantize(out=W, dtype=dtype)
        else:
            for b, o0, o1 in zip(self.bases, self.offsets[:-1], self.offsets[1:]):
                b.dequantize(out=W[:, o0:o1], dtype=dtype)  # written in place through the row stride
        return W, True

    def lora_cat(self, dtype, device, reuse: bool = False):
        """(A_cat [R_pad, in], B_blk [total_out, R_pad], slices) with the scaling folded into B_blk; R is padded
        with zero rows/columns to a multiple of 8."""
        # the backward of a step asks for the same matrices as its forward built (``reuse``); a forward always
        # rebuilds them, so an optimizer that updates the adapters through a flat buffer is seen as well
        key = (dtype, tuple((id(p), p._version) for l in self.loras if l is not None for p in _lora_parts(l)[:2]))
        cached = getattr(self, "_lora_cat_cache", None)
        if reuse and cached is not None and cached[0] == key:
            return cached[1]
        As, R = [], 0
        slices = []
        for l in self.loras:
            if l is None:
                slices.append(None)
                continue
            A, B, s = _lora_parts(l)
            slices.append((R, R + A.shape[0], s))
            R += A.shape[0]
            As.append(A.to(dtype))
        Rp = (R + 7) // 8 * 8
        if Rp != R:
            As.append(torch.zeros(Rp - R, self.in_features, dtype=dtype, device=device))
        A_cat = As[0] if len(As) == 1 else torch.cat(As, dim=0)
        B_blk = torch.zeros(self.total_out, Rp, dtype=dtype, device=device)
        for l, sl, o0, o1 in zip(self.loras, slices, self.offsets[:-1], self.offsets[1:]):
            if l is None:
                continue
            _, B, s = _lora_parts(l)
            B_blk[o0:o1, sl[0]:sl[1]] = B.to(dtype) * s
        self._lora_cat_cache = (key, (A_cat, B_blk, slices))
        return A_cat, B_blk, slices

    # ------------------------------------------------------------------ forward
    def dropout_p(self) -> float:
        """LoRA input dropout of this group while training (0.0 in eval mode or without dropout)."""
        for l in self.loras:
            if l is None or not l.training:
                continue
            name = l.active_adapters[0] if hasattr(l, "active_adapters") else "default"
            d = l.lora_dropout[name] if hasattr(l, "lora_dropout") else None
            p = float(getattr(d, "p", 0.0)) if d is not None else 0.0
            if p > 0.0:
                return p
        return 0.0

    def dropout_module(self):
        """A dropout module other than ``nn.Dropout`` / ``nn.Identity`` on the group's adapters while training (e.g. one
        that applies a fixed mask), else None.  Such a module is asked once for its element-wise factor,
        ``module(ones_like(x))``, which then serves the whole group (the reference calls the module on the input and
        reads the mask back from the zeros, fused_ops/unsloth_lora/bnb/fast_lora.py:262-288, 339-352)."""
        for l in self.loras:
            if l is None or not l.training or not hasattr(l, "lora_dropout"):
                continue
            name = l.active_adapters[0] if hasattr(l, "active_adapters") else "default"
            d = l.lora_dropout[name]
            if not isinstance(d, (nn.Dropout, nn.Identity)):
                return d
        return None

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                aux: Optional[dict] = None):
        """x [T, in] -> (y [T, total_out], xa [T, R] or None).  ``residual`` is added in the GEMM epilogue.
        With LoRA dropout the keep mask is left in ``aux["mask"]`` for :meth:`backward` (the adapter branch sees
        ``dropout(x)``, the base branch sees ``x``, as in the reference's fused LoRA functions)."""
        dtype, dev = x.dtype, x.device
        xa = None
        a2 = b2 = None
        if self.has_lora:
            A_cat, B_blk, _ = self.lora_cat(dtype, dev)
            p = self.dropout_p()
            custom = self.dropout_module()
            if custom is not None:
                if aux is None:
                    raise ValueError("LoRA dropout is active: pass an `aux` dict to keep the mask for the backward")
                aux["mask"], aux["keep_scale"] = custom(torch.ones_like(x)), 1.0
                xa = gemm(x * aux["mask"], A_cat)
            elif p > 0.0:
                if aux is None:
                    raise ValueError("LoRA dropout is active: pass an `aux` dict to keep the mask for the backward")
                mask = torch.rand(x.shape, device=dev) >= p
                aux["mask"], aux["keep_scale"] = mask, 1.0 / (1.0 - p)
                xa = gemm(x * mask * aux["keep_scale"], A_cat)
            else:
                xa = gemm(x, A_cat)
            a2, b2 = xa, B_blk
        beta = 1.0 if residual is not None else 0.0
        if self.kind == "dense" and len(self.bases) > 1:
            y = out if out is not None else torch.empty(x.shape[0], self.total_out, dtype=dtype, device=dev)
            for b, o0, o1 in zip(self.bases, self.offsets[:-1], self.offsets[1:]):
                gemm(x, b.weight, a2=a2, b2=(b2[o0:o1] if b2 is not None else None),
                     c=(residual[:, o0:o1] if residual is not None else None), beta=beta, out=y[:, o0:o1])
            return y, xa
        W, b_mn = self.dense_weight(dtype, dev)
        if b_mn and b2 is not None:
            b2 = b2.t().contiguous()  # second pair must share the orientation of the first
        y = gemm(x, W, b_mn=b_mn, a2=a2, b2=b2, c=residual, beta=beta, out=out)
        return y, xa

    # ------------------------------------------------------------------ backward
    def backward(self, dy: torch.Tensor, x: torch.Tensor, xa: Optional[torch.Tensor], need_dx: bool = True,
                 dx_residual: Optional[torch.Tensor] = None, aux: Optional[dict] = None):
        """Returns (dx [T, in] or None, grads aligned with ``trainable()``).  ``dx_residual`` is added to dx."""
        dtype, dev = dy.dtype, dy.device
        grads: List[torch.Tensor] = []
        dxa_s = None
        A_cat = None
        mask = aux.get("mask") if aux else None
        if self.has_lora:
            A_cat, B_blk, slices = self.lora_cat(dtype, dev, reuse=True)
            R = A_cat.shape[0]
            # dxa = dy @ B_blk  (already carries the scaling)
            dxa_s = gemm(dy, B_blk, b_mn=True)
            # dB_blk = dy^T @ xa ; dA_cat = dxa^T @ dropout(x)
            dB_blk = gemm(dy, xa, a_mn=True, b_mn=True, out_dtype=torch.float32)
            xd = x if mask is None else x * mask * aux["keep_scale"]
            dA_cat = gemm(dxa_s, xd, a_mn=True, b_mn=True, out_dtype=torch.float32)
        dx = None
        if need_dx:
            beta = 1.0 if dx_residual is not None else 0.0
            # with dropout the adapter's input gradient is masked, so it cannot ride on the base GEMM
            a2 = dxa_s if (self.has_lora and mask is None) else None
            if self.kind == "dense" and len(self.bases) > 1:
                dx = torch.empty(dy.shape[0], self.in_features, dtype=dtype, device=dev)
                first = True
                for b, o0, o1 in zip(self.bases, self.offsets[:-1], self.offsets[1:]):
                    gemm(dy[:, o0:o1], b.weight, b_mn=True,
                         a2=(a2 if first else None), b2=(A_cat if (first and a2 is not None) else None),
                         c=(dx_residual if first else dx), beta=(beta if first else 1.0), out=dx)
                    first = False
            else:
                W, w_mn = self.dense_weight(dtype, dev)
                # dx = dy @ W : W [out,in] is the [K,N] (MN-major) operand; a GPTQ W [in,out] is K-major here
                if w_mn:
                    b2 = A_cat.t().contiguous() if a2 is not None else None
                    dx = gemm(dy, W, b_mn=False, a2=a2, b2=b2, c=dx_residual, beta=beta)
                else:
                    dx = gemm(dy, W, b_mn=True, a2=a2, b2=A_cat, c=dx_residual, beta=beta)
            if mask is not None:
                dxl = gemm(dxa_s, A_cat, b_mn=True)  # [T, in]
                dx = torch.addcmul(dx, dxl, mask.to(dtype), value=aux["keep_scale"])
        # parameter gradients in the order of trainable()
        for i, (b, l) in enumerate(zip(self.bases, self.loras)):
            o0, o1 = self.offsets[i], self.offsets[i + 1]
            if self.kind == "dense" and b.weight.requires_grad:
                grads.append(gemm(dy[:, o0:o1], x, a_mn=True, b_mn=True, out_dtype=torch.float32))
            if l is not None:
                r0, r1, s = slices[i]
                A, B, _ = _lora_parts(l)
                grads.append(dA_cat[r0:r1].to(A.dtype))
                # xa is unscaled, so dB = s * dy^T xa
                grads.append((dB_blk[o0:o1, r0:r1] * s).to(B.dtype))
        return dx, grads
