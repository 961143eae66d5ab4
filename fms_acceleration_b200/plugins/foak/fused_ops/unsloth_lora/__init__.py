"""``fms_acceleration_foak.fused_ops.unsloth_lora``: fused LoRA projections and gated activations.  The reference's
three autograd functions per base type (``LoRA_QKV``, ``LoRA_W``, ``LoRA_MLP``) are one mechanism here, the
projection group of ``fms_acceleration_b200.ops.proj``."""
