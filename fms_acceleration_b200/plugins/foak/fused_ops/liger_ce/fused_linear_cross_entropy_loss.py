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
