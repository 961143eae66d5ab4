"""Rules for Hugging Face ``transformers`` model classes (llama, mistral, granite, mixtral, granitemoe,
granitemoeshared, granitemoehybrid, gpt_bigcode), built lazily and only when the class can be imported.

Per architecture (as in the reference, fms_acceleration_foak/models/*.py):
  ``-rms``          RMSNorm.forward -> fused kernel
  ``-rope``         ``apply_rotary_pos_emb`` of the modeling module -> fused kernel (import + reload)
  ``-qkvo``         attention: q/k/v (one fused call, K and V cached for the following two) and o projections
  ``-mlp``          gated MLP with LoRA on its three projections (only when the activation is SiLU)
  ``-custom-loss``  ``LOSS_MAPPING`` entry -> fast causal-LM loss;  ``-cross-ent`` for old transformers
  ``-fused-lce``    ``*ForCausalLM.forward`` -> chunked fused linear + cross-entropy
"""
from __future__ import annotations

import importlib
from functools import partial
from typing import List


from ....framework.model_patcher import (ModelPatcherRule, ModelPatcherTrigger, combine_functions, combine_triggers)
from ....ops.cross_entropy import FastCrossEntropyLoss, causal_lm_loss, fused_linear_cross_entropy
from ....ops.rmsnorm import fast_rms_layernorm
from ....ops.rope import fast_rope_embedding
from .utils import build_lora_fused_ops, trigger_fused_ops

# arch key -> (modeling module, class prefix, has dense gated MLP)
ARCHS = {
    "llama": ("transformers.models.llama.modeling_llama", "Llama", True),
    "mistral": ("transformers.models.mistral.modeling_mistral", "Mistral", True),
    "granite": ("transformers.models.granite.modeling_granite", "Granite", True),
    "mixtral": ("transformers.models.mixtral.modeling_mixtral", "Mixtral", False),
    "granitemoe": ("transformers.models.granitemoe.modeling_granitemoe", "GraniteMoe", False),
    "granitemoeshared": ("transformers.models.granitemoeshared.modeling_granitemoeshared", "GraniteMoeShared", False),
    "granitemoehybrid": ("transformers.models.granitemoehybrid.modeling_granitemoehybrid", "GraniteMoeHybrid", False),
    "gpt_bigcode": ("transformers.models.gpt_bigcode.modeling_gpt_bigcode", "GPTBigCode", False),
}


def _try_import(path: str):
    try:
        return importlib.import_module(path)
    except Exception:  # transformers absent or the family not present in this version
        return None


def _fast_causal_lm_loss(logits, labels, vocab_size=None, num_items_in_batch=None, ignore_index=-100, **kwargs):
    return causal_lm_loss(logits, labels, num_items_in_batch=num_items_in_batch, ignore_index=ignore_index)


def replace_custom_loss_when_triggered(model_cls, custom_loss_type: str):
    """Trigger that installs the fast loss into transformers' ``LOSS_MAPPING`` and points the model at it."""
    def _trigger(module):
        if isinstance(module, model_cls):
            lu = _try_import("transformers.loss.loss_utils")
            if lu is not None:
                lu.LOSS_MAPPING[custom_loss_type] = _fast_causal_lm_loss
                module.loss_type = custom_loss_type
            return True
        return False

    return _trigger


def lce_forward(self, input_ids=None, attention_mask=None, position_ids=None, past_key_values=None, inputs_embeds=None,
                labels=None, num_items_in_batch=None, **kwargs):
    """Replacement ``*ForCausalLM.forward``: in training the logits are never materialised."""
    outputs = self.model(input_ids=input_ids, attention_mask=attention_mask, position_ids=position_ids,
                         past_key_values=past_key_values, inputs_embeds=inputs_embeds, **kwargs)
    hidden = outputs[0]
    loss = logits = None
    if self.training and labels is not None:
        shift_h = hidden[..., :-1, :].reshape(-1, hidden.shape[-1])
        shift_l = labels[..., 1:].reshape(-1)
        scale = getattr(self.config, "logits_scaling", None)
        if scale:
            shift_h = shift_h / scale
        loss = fused_linear_cross_entropy(shift_h.contiguous(), self.lm_head.weight, shift_l.contiguous(),
                                          num_items=num_items_in_batch)
    else:
        logits = self.lm_head(hidden)
        if labels is not None:
            loss = causal_lm_loss(logits, labels, num_items_in_batch=num_items_in_batch)
    try:
        from transformers.modeling_outputs import CausalLMOutputWithPast

        return CausalLMOutputWithPast(loss=loss, logits=logits, past_key_values=getattr(outputs, "past_key_values", None))
    except Exception:
        return (loss, logits)


def get_mp_rules(arch: str, base_type: str, config=None) -> List[ModelPatcherRule]:
    path, prefix, dense_mlp = ARCHS[arch]
    mod = _try_import(path)
    if mod is None:
        return []
    rules: List[ModelPatcherRule] = []
    norm_cls = getattr(mod, f"{prefix}RMSNorm", None)
    attn_cls = getattr(mod, f"{prefix}Attention", None)
    mlp_cls = getattr(mod, f"{prefix}MLP", None)
    lm_cls = getattr(mod, f"{prefix}ForCausalLM", None)

    if norm_cls is not None:
        rules.append(ModelPatcherRule(rule_id=f"{arch}-rms", trigger=ModelPatcherTrigger(check=norm_cls),
                                      forward=fast_rms_layernorm))
    if attn_cls is not None and arch != "gpt_bigcode":
        rules.append(ModelPatcherRule(
            rule_id=f"{arch}-qkvo",
            trigger=combine_triggers(
                ModelPatcherTrigger(check=partial(trigger_fused_ops, attn_cls=attn_cls,
                                                  submodule_names=["q_proj", "k_proj", "v_proj"])),
                ModelPatcherTrigger(check=partial(trigger_fused_ops, attn_cls=attn_cls, submodule_names=["o_proj"])),
                logic="OR"),
            forward_builder=combine_functions(
                partial(build_lora_fused_ops, submodule_names=["q_proj", "k_proj", "v_proj"], fused_op="qkv",
                        base_type=base_type),
                partial(build_lora_fused_ops, submodule_names=["o_proj"], fused_op="o", base_type=base_type),
                logic="APPEND")))
    act = getattr(config, "hidden_act", None) if config is not None else None
    if dense_mlp and mlp_cls is not None and (act is None or act == "silu"):
        rules.append(ModelPatcherRule(
            rule_id=f"{arch}-mlp",
            trigger=ModelPatcherTrigger(check=partial(trigger_fused_ops, attn_cls=mlp_cls,
                                                      submodule_names=["up_proj", "down_proj", "gate_proj"])),
            forward_builder=partial(build_lora_fused_ops, submodule_names=["up_proj", "down_proj", "gate_proj"],
                                    fused_op="mlp", base_type=base_type)))
    if hasattr(mod, "apply_rotary_pos_emb"):
        rules.append(ModelPatcherRule(rule_id=f"{arch}-rope",
                                      import_and_maybe_reload=(f"{path}.apply_rotary_pos_emb", fast_rope_embedding, None)))
    if lm_cls is not None:
        if _try_import("transformers.loss.loss_utils") is not None:
            rules.append(ModelPatcherRule(
                rule_id=f"{arch}-custom-loss",
                trigger=ModelPatcherTrigger(check=replace_custom_loss_when_triggered(lm_cls, f"{arch}_custom_loss"))))
        else:
            rules.append(ModelPatcherRule(
                rule_id=f"{arch}-cross-ent",
                import_and_maybe_reload=("torch.nn.CrossEntropyLoss", FastCrossEntropyLoss, path)))
        if arch != "gpt_bigcode":
            rules.append(ModelPatcherRule(rule_id=f"{arch}-fused-lce", trigger=ModelPatcherTrigger(check=lm_cls),
                                          forward=lce_forward))
    return rules
