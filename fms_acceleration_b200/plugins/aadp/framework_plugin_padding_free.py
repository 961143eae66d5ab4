"""Padding-free plugin - configuration path ``training.attention.padding_free`` (``method: huggingface``).

What the reference does (fms_acceleration_aadp/framework_plugin_padding_free.py:30-243): replace the training
collator by one that flattens the mini-batch (``DataCollatorForSeq2Seq`` -> ``DataCollatorWithFlattening``;
a completion-only collator gets its padding stripped), and make attention honour document boundaries derived
from ``position_ids``.  Here the attention side is this package's own varlen kernel: in-tree models consume
``position_ids`` / ``cu_seqlens`` natively, and for Hugging Face models a patch rule swaps
``_flash_attention_forward`` for an adapter onto the same kernel.
"""
from __future__ import annotations

from typing import Dict, Tuple


from ...framework.framework_plugin import AccelerationPlugin
from .aadp_utils import DataCollatorWithFlattening, patch_torch_call_remove_padding


def _unwrap_collator(collate_fn):
    """HF Trainer may wrap the user's collator in a ``RemoveColumnsCollator``."""
    inner = getattr(collate_fn, "data_collator", None)
    return inner if inner is not None and collate_fn.__class__.__name__ == "RemoveColumnsCollator" else collate_fn


class PaddingFreeAccelerationPlugin(AccelerationPlugin):
    # the varlen attention kernel is in-tree; flash_attn is not needed
    require_packages = None

    def __init__(self, configurations: Dict[str, Dict]):
        super().__init__(configurations)
        self._method = self._check_config_and_maybe_check_values(
            key="training.attention.padding_free.method", values=["huggingface"])

    @property
    def requires_augmentation(self):
        return True

    def augmentation(self, model, train_args, modifiable_args: Tuple):
        from ...framework.accelerator_patcher import AcceleratorPatcher, AcceleratorPatcherComponent
        from ...framework.model_patcher import ModelPatcher, ModelPatcherRule

        def _collator_check(collate_fn) -> bool:
            name = _unwrap_collator(collate_fn).__class__.__name__
            return name in ("DataCollatorForSeq2Seq", "DataCollatorForCompletionOnlyLM", "DataCollatorWithFlattening",
                            "DataCollatorWithPadding", "function", "DefaultDataCollator")

        def _collator_replacement_builder(collate_fn):
            inner = _unwrap_collator(collate_fn)
            name = inner.__class__.__name__
            if name == "DataCollatorForCompletionOnlyLM":
                if hasattr(inner, "padding_free"):
                    inner.padding_free = True
                else:
                    patch_torch_call_remove_padding(inner)
                replacement = inner
            elif name == "DataCollatorWithFlattening":
                replacement = inner
            else:
                replacement = DataCollatorWithFlattening()
            if inner is not collate_fn:  # keep the column-removing wrapper
                collate_fn.data_collator = replacement
                return collate_fn
            return replacement

        if "padding-free" not in {h.rule_id for h in AcceleratorPatcher.history}:
            AcceleratorPatcher.replace(
                "padding-free", AcceleratorPatcherComponent.data_collator,
                replacement_builder=_collator_replacement_builder, pre_requisite_check=_collator_check)

        if hasattr(train_args, "padding_free"):
            train_args.padding_free = True

        # Hugging Face models: attention goes to the in-tree varlen kernel, through the attention registry where
        # transformers has one, and through its flash-attention entry point for older versions
        if model.__class__.__module__.startswith("transformers.") or hasattr(getattr(model, "config", None),
                                                                             "_attn_implementation"):
            from .flash_attn import use_in_tree_attention

            use_in_tree_attention(model)
        try:
            import transformers.modeling_flash_attention_utils as fa_utils  # noqa: F401

            from .flash_attn import build_fa_forward

            if "flash-attn-varlen" not in ModelPatcher.rules:
                ModelPatcher.register(ModelPatcherRule(
                    rule_id="flash-attn-varlen",
                    import_and_maybe_reload=("transformers.modeling_flash_attention_utils._flash_attention_forward",
                                             build_fa_forward(), None)))
        except Exception:
            pass
        return model, modifiable_args


AccelerationPlugin.register_plugin(PaddingFreeAccelerationPlugin,
                                   configuration_and_paths=["training.attention.padding_free"])
