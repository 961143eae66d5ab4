"""Cross-entropy and chunked fused linear + cross-entropy (``csrc/cross_entropy.cu`` + tcgen05 GEMM).

Reference behaviour:
* fms_acceleration_foak/kernels/unsloth/cross_entropy_loss.py:190-343 - ``Fast_CrossEntropyLoss`` saves the
  logsumexp in the forward and overwrites the logits with their gradient in the backward;
  ``FastForCausalLMLoss`` shifts labels, ignores index -100 and divides by ``num_items_in_batch`` when given.
* fms_acceleration_foak/fused_ops/liger_ce/fused_linear_cross_entropy_loss.py:45-219 - the logits are never
  materialised for the whole batch: per chunk of rows ``logits = x W^T``, loss and dlogits in one kernel,
  ``dx = dlogits W`` and ``dW += dlogits^T x``.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .. import _native as N
from .gemm import gemm

IGNORE_INDEX = -100


def cross_entropy_ref(logits, labels, ignore_index=IGNORE_INDEX, label_smoothing=0.0):
    """Per-row losses (fp32), zeros at ignored rows."""
    return F.cross_entropy(logits.float(), labels.long(), ignore_index=ignore_index, reduction="none",
                           label_smoothing=label_smoothing)


def _labels64(labels):
    return labels if labels.dtype == torch.int64 else labels.long()


def ce_forward(logits2, labels, ignore_index=IGNORE_INDEX, label_smoothing=0.0, write_grad=False, scale=None,
               row_scale=None):
    """Launch the CE kernel on 2-D logits.  Returns (loss_rows, lse_rows).  With ``write_grad`` the logits are
    overwritten by ``scale * row_scale * dloss/dlogits``."""
    rows, V = logits2.shape
    loss = torch.empty(rows, dtype=torch.float32, device=logits2.device)
    lse = torch.empty(rows, dtype=torch.float32, device=logits2.device)
    rc = N.lib().fmsb_ce(logits2.data_ptr(), logits2.stride(0), labels.data_ptr(), loss.data_ptr(), lse.data_ptr(),
                         N.ptr(scale), N.ptr(row_scale), rows, V, ignore_index, float(label_smoothing),
                         int(write_grad), N.dtype_code(logits2.dtype), N.stream_ptr())
    N.check(rc, "fmsb_ce")
    return loss, lse


def count_valid(labels, ignore_index=IGNORE_INDEX):
    """Device tensor [count, 1/max(count,1)] of labels != ignore_index (no host sync)."""
    out = torch.empty(2, dtype=torch.float32, device=labels.device)
    rc = N.lib().fmsb_count_valid(labels.data_ptr(), labels.numel(), ignore_index, out.data_ptr(), N.stream_ptr())
    N.check(rc, "fmsb_count_valid")
    return out


class _CrossEntropy(torch.autograd.Function):
    """Per-row CE; the backward writes the gradient over the logits storage (as the reference does)."""

    @staticmethod
    def forward(ctx, logits, labels, ignore_index, inplace_backward):
        V = logits.shape[-1]
        l2 = logits.reshape(-1, V)
        if l2.stride(1) != 1:
            l2 = l2.contiguous()
        lab = _labels64(labels.reshape(-1)).contiguous()
        loss, lse = ce_forward(l2, lab, ignore_index)
        ctx.save_for_backward(l2, lab, lse)
        ctx.ignore_index = ignore_index
        ctx.inplace = inplace_backward
        ctx.shape = logits.shape
        return loss.view(labels.shape)

    @staticmethod
    def backward(ctx, dloss):
        l2, lab, lse = ctx.saved_tensors
        g = l2 if ctx.inplace else torch.empty_like(l2)
        d = dloss.reshape(-1).float().contiguous()
        rc = N.lib().fmsb_ce_bwd(l2.data_ptr(), l2.stride(0), g.data_ptr(), g.stride(0), lab.data_ptr(),
                                 lse.data_ptr(), d.data_ptr(), 1, g.shape[0], g.shape[1], ctx.ignore_index,
                                 N.dtype_code(g.dtype), N.stream_ptr())
        N.check(rc, "fmsb_ce_bwd")
        return g.view(ctx.shape), None, None, None


def fast_cross_entropy_loss(logits, labels, ignore_index=IGNORE_INDEX, inplace_backward=True):
    """Per-token losses with the shape of ``labels``."""
    if not logits.is_cuda:
        return cross_entropy_ref(logits.reshape(-1, logits.shape[-1]), labels.reshape(-1), ignore_index).view(labels.shape)
    return _CrossEntropy.apply(logits, labels, ignore_index, inplace_backward)


def causal_lm_loss(logits, labels, num_items_in_batch=None, ignore_index=IGNORE_INDEX, shift=True):
    """Same contract as ``FastForCausalLMLoss`` (reference cross_entropy_loss.py:299-324)."""
    if shift:
        logits = logits[..., :-1, :]
        labels = labels[..., 1:]
    per_tok = fast_cross_entropy_loss(logits, labels.contiguous(), ignore_index)
    if num_items_in_batch is None:
        n = (labels != ignore_index).sum().clamp(min=1)
    else:
        n = num_items_in_batch
    return per_tok.sum() / n


class FastCrossEntropyLoss(torch.nn.CrossEntropyLoss):
    """Drop-in for ``torch.nn.CrossEntropyLoss`` (mean over non-ignored targets)."""

    def forward(self, input, target):
        per_tok = fast_cross_entropy_loss(input, target, self.ignore_index)
        n = (target != self.ignore_index).sum().clamp(min=1)
        return per_tok.sum() / n


# ------------------------------------------------------------------------------------------------
# fused linear + CE
# ------------------------------------------------------------------------------------------------
def fused_linear_ce_ref(x, weight, labels, ignore_index=IGNORE_INDEX, num_items=None, label_smoothing=0.0):
    logits = x.float() @ weight.float().t()
    per = cross_entropy_ref(logits, labels, ignore_index, label_smoothing)
    n = (labels != ignore_index).sum().clamp(min=1) if num_items is None else num_items
    return per.sum() / n


def _chunk_rows(rows: int, V: int, elem_bytes: int, budget_bytes: int = 512 << 20) -> int:
    c = max(128, (budget_bytes // (V * elem_bytes)) // 128 * 128)
    return min(rows, c)


class _FusedLinearCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, labels, ignore_index, num_items, label_smoothing, need_dw):
        # x [T, H] (16-bit), weight [V, H], labels [T]
        T, H = x.shape
        V = weight.shape[0]
        lab = _labels64(labels).contiguous()
        if num_items is None:
            cnt = count_valid(lab, ignore_index)
            scale = cnt[1:2]
        else:
            scale = torch.full((1,), 1.0 / float(num_items), dtype=torch.float32, device=x.device) \
                if not torch.is_tensor(num_items) else (1.0 / num_items.float().reshape(1))
        dx = torch.empty_like(x)
        dw = torch.zeros(V, H, dtype=torch.float32, device=x.device) if need_dw else None
        loss_rows = torch.empty(T, dtype=torch.float32, device=x.device)
        C = _chunk_rows(T, V, x.element_size())
        # rows of the logits chunk start on 16-byte boundaries whatever the vocabulary size (49155 for Granite)
        logits = torch.empty(C, (V + 7) // 8 * 8, dtype=x.dtype, device=x.device)
        for s in range(0, T, C):
            e = min(T, s + C)
            lg = logits[: e - s, :V]
            gemm(x[s:e], weight, out=lg)
            l, _ = ce_forward(lg, lab[s:e], ignore_index, label_smoothing, write_grad=True, scale=scale)
            loss_rows[s:e] = l
            gemm(lg, weight, b_mn=True, out=dx[s:e])  # dx = dlogits @ W
            if need_dw:
                _accumulate_dw(dw, lg, x[s:e])  # dW[V,H] += dlogits^T[V,rows] @ x[rows,H]
        loss = loss_rows.sum() * scale[0]
        ctx.save_for_backward(dx, dw)
        ctx.wdtype = weight.dtype
        return loss

    @staticmethod
    def backward(ctx, dloss):
        dx, dw = ctx.saved_tensors
        gx = dx * dloss.to(dx.dtype)
        gw = None if dw is None else (dw * dloss).to(ctx.wdtype)
        return gx, gw, None, None, None, None, None


def _accumulate_dw(dw, dlogits, x):
    part = gemm(dlogits, x, a_mn=True, b_mn=True, out_dtype=torch.float32)
    dw.add_(part)


def fused_linear_cross_entropy(x, weight, labels, ignore_index=IGNORE_INDEX, num_items=None, label_smoothing=0.0):
    """Mean CE of ``x @ weight.T`` against ``labels`` without materialising all logits."""
    x2 = x.reshape(-1, x.shape[-1])
    lab = labels.reshape(-1)
    if not x2.is_cuda:
        return fused_linear_ce_ref(x2, weight, lab, ignore_index, num_items, label_smoothing)
    return _FusedLinearCE.apply(x2.contiguous(), weight, lab, ignore_index, num_items, label_smoothing,
                                weight.requires_grad)
