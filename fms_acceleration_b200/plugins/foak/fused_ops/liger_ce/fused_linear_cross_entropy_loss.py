"""Names of fms_acceleration_foak/fused_ops/liger_ce/fused_linear_cross_entropy_loss.py:221-418."""
import torch

from fms_acceleration_b200.ops.cross_entropy import _FusedLinearCE as LigerFusedLinearCrossEntropyFunction  # noqa: F401
from fms_acceleration_b200.ops.cross_entropy import fused_linear_ce_ref, fused_linear_cross_entropy  # noqa: F401
from fms_acceleration_b200.plugins.foak.models.hf import lce_forward  # noqa: F401


class LigerFusedLinearCrossEntropyLoss(torch.nn.CrossEntropyLoss):
    """``loss(lin_weight, hidden, target)`` as in the reference (:269-282); mean over the non-ignored targets."""

    def forward(self, lin_weight, _input, target, bias=None):
        if bias is not None:
            raise NotImplementedError("a bias on the output projection is not supported")
        return fused_linear_cross_entropy(_input, lin_weight, target, ignore_index=self.ignore_index,
                                          label_smoothing=self.label_smoothing)


def fused_linear_cross_entropy_forward(_input, weight, target, bias=None, ignore_index=-100, label_smoothing=0.0,
                                       reduction="mean"):
    """Functional form with the reference's contract (:45-170): returns ``(loss, grad_input, grad_weight, grad_bias)``,
    the gradients already formed for an upstream gradient of 1.  Rows are processed in chunks so that only a chunk of
    the logits exists at a time.  Stated with tensor ops (any device); the training path is
    :class:`LigerFusedLinearCrossEntropyFunction`, whose chunks run on the in-tree GEMM and cross-entropy kernels."""
    if reduction not in ("mean", "sum"):
        raise ValueError("reduction must be 'mean' or 'sum'")
    BT, H = _input.shape
    V = weight.shape[0]
    chunk = max(1, min(BT, (BT * H + V - 1) // V))  # a chunk of logits is about as large as the input
    valid = target != ignore_index
    denom = valid.sum().clamp(min=1).to(torch.float32) if reduction == "mean" else torch.ones((), device=_input.device)
    grad_input = torch.zeros_like(_input)
    grad_weight = torch.zeros_like(weight) if weight.requires_grad else None
    grad_bias = torch.zeros_like(bias) if bias is not None else None
    loss = torch.zeros((), dtype=torch.float32, device=_input.device)
    for s in range(0, BT, chunk):
        e = min(BT, s + chunk)
        x = _input[s:e]
        logits = (x @ weight.t()).float()
        if bias is not None:
            logits = logits + bias.float()
        tgt, ok = target[s:e], valid[s:e]
        logp = torch.log_softmax(logits, dim=-1)
        safe = tgt.clamp(min=0)
        nll = -logp.gather(1, safe[:, None]).squeeze(1)
        grad = logp.exp()
        if label_smoothing > 0:
            nll = (1 - label_smoothing) * nll - label_smoothing * logp.mean(dim=-1)
            grad = grad - label_smoothing / V
            grad.scatter_add_(1, safe[:, None], torch.full_like(nll, -(1 - label_smoothing))[:, None])
        else:
            grad.scatter_add_(1, safe[:, None], torch.full_like(nll, -1.0)[:, None])
        loss = loss + (nll * ok).sum()
        grad = (grad * ok[:, None] / denom).to(_input.dtype)
        grad_input[s:e] = grad @ weight
        if grad_weight is not None:
            grad_weight.add_((grad.t() @ x).to(grad_weight.dtype))
        if grad_bias is not None:
            grad_bias.add_(grad.sum(dim=0).to(grad_bias.dtype))
    return loss / denom, grad_input, grad_weight, grad_bias


def fused_linear_cross_entropy_backward(grad_output, grad_input, grad_weight, grad_bias):
    """Scale the gradients of :func:`fused_linear_cross_entropy_forward` by the upstream gradient (in place, as the
    reference does, :173-219)."""
    for g in (grad_input, grad_weight, grad_bias):
        if g is not None:
            g.mul_(grad_output.to(g.dtype))
    return grad_input, grad_weight, grad_bias
