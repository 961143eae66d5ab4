"""Quantised PEFT: NF4/FP4 QLoRA and GPTQ-LoRA."""
from .framework_plugin_bnb import BNBAccelerationPlugin  # noqa: F401
from .framework_plugin_autogptq import AutoGPTQAccelerationPlugin  # noqa: F401
