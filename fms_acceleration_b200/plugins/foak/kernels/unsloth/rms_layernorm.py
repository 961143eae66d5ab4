"""Names of fms_acceleration_foak/kernels/unsloth/rms_layernorm.py:131-192."""
from fms_acceleration_b200.ops.rmsnorm import _RMSNorm as Fast_RMS_Layernorm  # noqa: F401
from fms_acceleration_b200.ops.rmsnorm import fast_rms_layernorm, rmsnorm, rmsnorm_ref  # noqa: F401

__all__ = ["Fast_RMS_Layernorm", "fast_rms_layernorm", "rmsnorm", "rmsnorm_ref"]
