"""Fused-ops-and-kernels plugin, registered on ``training.fused_ops_and_kernels`` OR
``peft.quantization.fused_ops_and_kernels``.

Options, defaults, rule-id suffix filtering and the restricted architectures are those of
fms_acceleration_foak/framework_plugin_fast_kernels.py:77-222 in the reference:

    base_layer            auto_gptq | bitsandbytes      (default auto_gptq)
    fused_lora            bool -> rules ending in ``qkvo`` / ``mlp`` (dropped for unquantised models)
    fast_loss             False | True -> ``cross-ent`` / ``custom-loss`` | "fused_ce_liger" -> ``fused-lce``
    fast_rms_layernorm    bool -> ``rms``
    fast_rope_embeddings  bool -> ``rope``

For the in-tree model zoo the selected kernels are applied as whole-block fusions
(:mod:`fms_acceleration_b200.ops.fused_layer`); for Hugging Face model classes the same kernels are applied
module by module through ModelPatcher rules (``foak/models``).
"""
from __future__ import annotations

from typing import Dict, Set, Tuple

import torch

from ...framework.framework_plugin import AccelerationPlugin, AccelerationPluginConfigError
from .utils import filter_mp_rules, lora_adapters_switch_ddp_from_fsdp

FILTER_MAP = {
    "fused_lora": {"qkvo", "mlp"},
    "fast_loss": {True: {"cross-ent", "custom-loss"}, "fused_ce_liger": "fused-lce"},
    "fast_rms_layernorm": "rms",
    "fast_rope_embeddings": "rope",
}


def register_foak_model_patch_rules(base_type: str, filter_endswith: Set[str] = None, config=None) -> None:
    from ...framework.model_patcher import ModelPatcher
    from .models import all_rules

    rules = all_rules(base_type, config)
    if filter_endswith:
        rules = filter_mp_rules(rules, filter_endswith)
    for rule in rules:
        if rule.rule_id not in ModelPatcher.rules:
            ModelPatcher.register(rule)


class FastKernelsAccelerationPlugin(AccelerationPlugin):
    restricted_model_archs = [
        "GraniteForCausalLM", "GraniteMoeForCausalLM", "GPTBigCodeForCausalLM", "MixtralForCausalLM",
        "LlamaForCausalLM", "MistralForCausalLM", "GraniteMoeSharedForCausalLM", "GraniteMoeHybridForCausalLM",
        "Mamba2ForCausalLM",  # in-tree Mamba2: fused loss (its scan / conv / norm kernels are always the native ones)
    ]

    def __init__(self, configurations: Dict[str, Dict]):
        super().__init__(configurations)
        try:
            self.configurations = self._check_config_and_maybe_check_values(key="training.fused_ops_and_kernels")
        except AccelerationPluginConfigError:
            self.configurations = self._check_config_and_maybe_check_values(key="peft.quantization.fused_ops_and_kernels")
        c = self.configurations
        c["base_layer"] = self._check_config_and_maybe_check_values(
            key="base_layer", values=["auto_gptq", "bitsandbytes"], default="auto_gptq")
        c["fused_lora"] = self._check_config_and_maybe_check_values(key="fused_lora", values=[False, True], default=False)
        c["fast_loss"] = self._check_config_and_maybe_check_values(
            key="fast_loss", values=[False, True, "fused_ce_liger"], default=False)
        c["fast_rms_layernorm"] = self._check_config_and_maybe_check_values(
            key="fast_rms_layernorm", values=[False, True], default=False)
        c["fast_rope_embeddings"] = self._check_config_and_maybe_check_values(
            key="fast_rope_embeddings", values=[False, True], default=False)

    @property
    def requires_augmentation(self):
        return True

    def selected_terms(self, quantised: bool) -> Set[str]:
        omitted = set() if quantised else {"fused_lora"}
        terms: Set[str] = set()
        for k, v in self.configurations.items():
            if isinstance(v, bool) and v is False:
                continue
            if k in FILTER_MAP and k not in omitted:
                ts = FILTER_MAP[k]
                if isinstance(ts, dict):
                    ts = ts.get(v, set())
                if isinstance(ts, str):
                    ts = {ts}
                terms.update(ts)
        return terms

    def augmentation(self, model, train_args, modifiable_args: Tuple):
        has_quant = getattr(model, "quantization_method", None)
        if has_quant:
            assert train_args.bf16 is True or train_args.fp16 is True, (
                f"{self.__class__} requires mixed precision argument `--fp16` or `--bf16`")
        terms = self.selected_terms(has_quant is not None)
        register_foak_model_patch_rules(self.configurations["base_layer"], terms, getattr(model, "config", None))
        # in-tree models: switch the packed, block-fused execution path on
        base = model.get_base_model() if hasattr(model, "get_base_model") else model
        if hasattr(base, "enable_fused") and terms & {"qkvo", "mlp", "rms", "rope"}:
            fast_loss = self.configurations["fast_loss"]
            base.enable_fused(fast_loss=fast_loss)
        elif hasattr(base, "fast_loss"):
            base.fast_loss = self.configurations["fast_loss"]
        return model, modifiable_args

    def get_callbacks_and_ready_for_train(self, model: torch.nn.Module = None, accelerator=None):
        is_quantized = getattr(model, "quantization_method", None) if model is not None else None
        if (accelerator is not None and getattr(accelerator.state, "fsdp_plugin", None) is not None
                and is_quantized is not None):
            lora_mods = [m for m in model.modules() if hasattr(m, "lora_A") and hasattr(m, "lora_B")]
            lora_adapters_switch_ddp_from_fsdp(lora_mods, accelerator.state.fsdp_plugin)
        return []


AccelerationPlugin.register_plugin(
    FastKernelsAccelerationPlugin,
    configuration_or_paths=["training.fused_ops_and_kernels", "peft.quantization.fused_ops_and_kernels"],
)
