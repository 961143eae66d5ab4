"""``fms_acceleration_foak.kernels.unsloth``: the names of the reference's fast RMSNorm / RoPE / cross-entropy modules.
The implementations are the CUDA kernels of ``fms_acceleration_b200.ops`` (``csrc/elementwise.cu``,
``csrc/cross_entropy.cu``); nothing here is Triton."""
from .cross_entropy_loss import fast_cross_entropy_loss  # noqa: F401,E402
from .rms_layernorm import fast_rms_layernorm  # noqa: F401,E402
from .rope_embedding import fast_rope_embedding  # noqa: F401,E402
