"""LoRA on GPTQ ``QuantLinear`` layers (role of fms_acceleration_peft/gptqmodel/utils/peft.py:41-169)."""
from __future__ import annotations

from typing import List

import torch

from fms_acceleration_b200.nn.gptq import QuantLinear
from fms_acceleration_b200.nn.lora import LoraConfig, LoraLinear, PeftModelShim


class GPTQLoraLinear(LoraLinear):
    """LoRA wrapper whose base layer is a GPTQ ``QuantLinear`` (never merged: the base is packed integers)."""

    def merge(self, *a, **k):
        raise NotImplementedError("a LoRA adapter cannot be merged into a GPTQ-packed weight")


def find_all_linear_names(model: torch.nn.Module, ignore: List[str] | None = None, ignore_lm_head: bool = True) -> List[str]:
    ignore = list(ignore or [])
    if ignore_lm_head and "lm_head" not in ignore:
        ignore.append("lm_head")
    names = set()
    for n, m in model.named_modules():
        if isinstance(m, QuantLinear):
            leaf = n.split(".")[-1]
            if leaf not in ignore:
                names.add(leaf)
    return sorted(names)


def get_gptq_peft_model(model, peft_config: LoraConfig = None, model_id: str = None, adapter_name: str = "default",
                        auto_find_all_linears: bool = True, train_mode: bool = False):
    if train_mode and peft_config is None:
        raise ValueError("peft_config not specified when in train mode.")
    if auto_find_all_linears:
        peft_config.target_modules = find_all_linear_names(model, ignore_lm_head=True)
    return PeftModelShim(model, peft_config, adapter_name)
