"""The reference's ``liger_cross_entropy_kernel`` computes the loss and, in the same pass, overwrites the logits with
their gradient (fms_acceleration_foak/fused_ops/liger_ce/cross_entropy.py:32-179).  The in-tree kernel does the same
(``csrc/cross_entropy.cu``, online log-sum-exp, label smoothing, device-side mean scale); this is its Python entry."""
from fms_acceleration_b200.ops.cross_entropy import ce_forward, cross_entropy_ref  # noqa: F401


def liger_cross_entropy(logits, labels, ignore_index: int = -100, label_smoothing: float = 0.0, scale=None):
    """Per-row losses; ``logits`` is overwritten with ``scale * d loss / d logits``."""
    loss, _ = ce_forward(logits, labels, ignore_index, label_smoothing, write_grad=True, scale=scale)
    return loss
