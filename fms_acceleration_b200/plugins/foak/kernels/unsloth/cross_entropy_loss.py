"""Names of fms_acceleration_foak/kernels/unsloth/cross_entropy_loss.py:192-343."""
from fms_acceleration_b200.ops.cross_entropy import _CrossEntropy as Fast_CrossEntropyLoss  # noqa: F401
from fms_acceleration_b200.ops.cross_entropy import FastCrossEntropyLoss, causal_lm_loss, fast_cross_entropy_loss  # noqa: F401
from fms_acceleration_b200.plugins.foak.models.hf import replace_custom_loss_when_triggered  # noqa: F401


def FastForCausalLMLoss(logits, labels, vocab_size: int = None, num_items_in_batch: int = None,
                        ignore_index: int = -100, **kwargs):
    """Shifted next-token loss, divided by ``num_items_in_batch`` when given (reference :299-324)."""
    return causal_lm_loss(logits, labels, num_items_in_batch=num_items_in_batch, ignore_index=ignore_index)


__all__ = ["Fast_CrossEntropyLoss", "FastCrossEntropyLoss", "FastForCausalLMLoss", "fast_cross_entropy_loss",
           "replace_custom_loss_when_triggered"]
