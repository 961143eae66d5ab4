"""Rules for the in-tree model zoo.

The zoo models execute the selected kernels as whole-block fusions once ``enable_fused`` has been called, so
most of these rules are markers (trigger only, no forward swap) that make the patch summary show what is
active; the RMSNorm rule really swaps the module forward so that norms outside the fused blocks (and the
eager path on a GPU) use the kernel too.
"""
from __future__ import annotations

from typing import List

from ....framework.model_patcher import ModelPatcherRule, ModelPatcherTrigger
from ....ops.rmsnorm import fast_rms_layernorm


def get_mp_rules(base_type: str, config=None) -> List[ModelPatcherRule]:
    from ....models import llama as L

    def _norm_forward(self, x):
        return fast_rms_layernorm(self, x)

    rules = [
        ModelPatcherRule(rule_id="zoo-rms", trigger=ModelPatcherTrigger(check=L.LlamaRMSNorm), forward=_norm_forward),
        ModelPatcherRule(rule_id="zoo-qkvo", trigger=ModelPatcherTrigger(check=L.LlamaAttention)),
        ModelPatcherRule(rule_id="zoo-rope", trigger=ModelPatcherTrigger(
            check=lambda m: isinstance(m, L.LlamaModel))),
        ModelPatcherRule(rule_id="zoo-fused-lce", trigger=ModelPatcherTrigger(
            check=lambda m: isinstance(m, L.LlamaForCausalLM) and m.fast_loss == "fused_ce_liger")),
        ModelPatcherRule(rule_id="zoo-cross-ent", trigger=ModelPatcherTrigger(
            check=lambda m: isinstance(m, L.LlamaForCausalLM) and m.fast_loss is True)),
    ]
    act = getattr(config, "hidden_act", "silu") if config is not None else "silu"
    if act == "silu":
        rules.append(ModelPatcherRule(rule_id="zoo-mlp", trigger=ModelPatcherTrigger(check=L.LlamaMLP)))
    return rules
