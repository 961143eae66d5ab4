"""Fused LoRA on 4-bit (NF4 / FP4) base weights."""
from .fast_lora import (apply_lora_mlp_geglu_approx, apply_lora_mlp_geglu_exact, apply_lora_mlp_swiglu,  # noqa: F401,E402
                        apply_lora_o, apply_lora_qkv, get_lora_parameters)
