"""Names of fms_acceleration_foak/fused_ops/unsloth_lora/bnb/fast_lora.py:21-471."""
from .._apply import (LoRA_MLP, LoRA_QKV, LoRA_W, apply_lora_mlp_geglu_approx, apply_lora_mlp_geglu_exact,  # noqa: F401
                      apply_lora_mlp_swiglu, apply_lora_o, apply_lora_o_v2, apply_lora_qkv)
from ..utils import fast_dequantize, get_lora_parameters, matmul_lora  # noqa: F401
