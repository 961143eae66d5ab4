"""LoRA on GPTQ ``QuantLinear`` layers (role of fms_acceleration_peft/gptqmodel/utils/peft.py:41-169)."""
from __future__ import annotations

import contextlib
from dataclasses import dataclass
from typing import List

import torch

from fms_acceleration_b200.nn.gptq import QuantLinear
from fms_acceleration_b200.nn.lora import LoraConfig, LoraLinear, PeftModelShim


@dataclass
class GPTQLoraConfig(LoraConfig):
    """``LoraConfig`` with the two switches of the reference's GPTQ LoRA configuration
    (fms_acceleration_peft/gptqmodel/utils/peft.py:41-43); both describe fused modules injected by other GPTQ
    back-ends and are only carried along here."""

    injected_fused_attention: bool = False
    injected_fused_mlp: bool = False


class GPTQLoraLinear(LoraLinear):
    """LoRA wrapper whose base layer is a GPTQ ``QuantLinear`` (never merged: the base is packed integers)."""

    def merge(self, *a, **k):
        raise NotImplementedError("a LoRA adapter cannot be merged into a GPTQ-packed weight")


class GPTQLoraModel(PeftModelShim):
    """LoRA model whose targets are GPTQ ``QuantLinear`` layers: every wrapped layer is a :class:`GPTQLoraLinear`
    and adapters are never merged (fms_acceleration_peft/gptqmodel/utils/peft.py:41-85)."""

    def __init__(self, model, peft_config: LoraConfig, adapter_name: str = "default"):
        super().__init__(model, peft_config, adapter_name)
        for mod in self.base_model.modules():
            if type(mod) is LoraLinear and isinstance(mod.base_layer, QuantLinear):
                mod.__class__ = GPTQLoraLinear

    def merge_adapter(self):
        raise NotImplementedError("GPTQ LoRA adapters cannot be merged")

    def unmerge_adapter(self):
        raise NotImplementedError("GPTQ LoRA adapters cannot be merged")

    def merge_and_unload(self):
        raise NotImplementedError("GPTQ LoRA adapters cannot be merged")


#: peft-type name -> model class used while :func:`hijack_peft_mappings` is active
PEFT_TYPE_TO_MODEL_MAPPING = {"LORA": PeftModelShim}


@contextlib.contextmanager
def hijack_peft_mappings():
    """While active, LoRA models are built as :class:`GPTQLoraModel` (with PEFT installed, PEFT's own type map is
    redirected as well); the previous mapping is restored on exit
    (fms_acceleration_peft/gptqmodel/utils/peft.py:88-104)."""
    saved = dict(PEFT_TYPE_TO_MODEL_MAPPING)
    PEFT_TYPE_TO_MODEL_MAPPING["LORA"] = GPTQLoraModel
    peft_map = peft_saved = None
    try:
        from peft.peft_model import PEFT_TYPE_TO_MODEL_MAPPING as peft_map  # type: ignore
        from peft.utils.peft_types import PeftType  # type: ignore

        peft_saved = peft_map.get(PeftType.LORA)
        peft_map[PeftType.LORA] = GPTQLoraModel
    except Exception:  # PEFT is optional
        peft_map = None
    try:
        yield
    finally:
        PEFT_TYPE_TO_MODEL_MAPPING.clear()
        PEFT_TYPE_TO_MODEL_MAPPING.update(saved)
        if peft_map is not None:
            from peft.utils.peft_types import PeftType  # type: ignore

            peft_map[PeftType.LORA] = peft_saved


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
    with hijack_peft_mappings():
        return PEFT_TYPE_TO_MODEL_MAPPING["LORA"](model, peft_config, adapter_name)
