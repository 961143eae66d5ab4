"""Names of fms_acceleration_foak/kernels/unsloth/rope_embedding.py:75-139.  Unlike the reference's kernel this one
honours ``position_ids`` (packed batches)."""
from fms_acceleration_b200.ops.rope import _Rope as Fast_RoPE_Embedding  # noqa: F401
from fms_acceleration_b200.ops.rope import apply_rope, fast_rope_embedding, rope_ref  # noqa: F401

__all__ = ["Fast_RoPE_Embedding", "fast_rope_embedding", "apply_rope", "rope_ref"]
