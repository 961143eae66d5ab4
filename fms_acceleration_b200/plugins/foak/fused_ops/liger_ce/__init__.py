"""``fms_acceleration_foak.fused_ops.liger_ce``: chunked linear + cross-entropy (the logits never exist as a whole)."""
from .fused_linear_cross_entropy_loss import (LigerFusedLinearCrossEntropyFunction,  # noqa: F401
                                              LigerFusedLinearCrossEntropyLoss, lce_forward)
