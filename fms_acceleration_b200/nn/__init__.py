"""Modules: quantised linears, LoRA wrappers."""
from .linear4bit import Linear4bit  # noqa: F401
from .lora import LoraConfig, LoraLinear, get_peft_model, PeftModelShim  # noqa: F401
