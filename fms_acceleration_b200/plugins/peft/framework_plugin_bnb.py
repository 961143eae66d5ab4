"""4-bit (NF4 / FP4, double-quantised) QLoRA plugin - configuration path ``peft.quantization.bitsandbytes``.

Same lifecycle as fms_acceleration_peft/framework_plugin_bnb.py:95-268 of the reference: a custom model
loader that produces a model whose linear layers are 4-bit, an augmentation that freezes the base, installs
the LoRA adapters and returns ``peft_config=None``, and the tied-weights fix at callback time.  The
quantisation itself is this package's own (``Linear4bit`` + ``csrc/quant.cu``): every decoder layer is
quantised right after it is built, so the 16-bit model never exists as a whole.
"""
from __future__ import annotations

import warnings
from typing import Dict, Tuple

import torch

from ...framework.framework_plugin import AccelerationPlugin
from ...models.builder import build_model, quantize_linears_
from ...nn.linear4bit import Linear4bit
from ...nn.lora import get_peft_model
from .fsdp_utils import ensure_weights_retied


def _prepare_model_for_kbit_training(model, use_gradient_checkpointing=True, gradient_checkpointing_kwargs=None):
    """Freeze the base model; no fp32 upcast of norms or embeddings (the reference avoids peft's stock
    ``prepare_model_for_kbit_training`` for that reason, framework_plugin_bnb.py:41-92)."""
    for p in model.parameters():
        p.requires_grad_(False)
    if use_gradient_checkpointing and hasattr(model, "gradient_checkpointing_enable"):
        if hasattr(model, "enable_input_require_grads"):
            model.enable_input_require_grads()
        model.gradient_checkpointing_enable(**({"gradient_checkpointing_kwargs": gradient_checkpointing_kwargs}
                                               if gradient_checkpointing_kwargs else {}))
    return model


class BNBAccelerationPlugin(AccelerationPlugin):
    # the quantiser is in-tree: nothing external is required
    require_packages = None

    def __init__(self, configurations: Dict[str, Dict]):
        super().__init__(configurations)
        self._quant_type = self._check_config_and_maybe_check_values(
            key="peft.quantization.bitsandbytes.quant_type", values=["fp4", "nf4"])
        self._no_peft_model = self._check_config_and_maybe_check_values(
            key="peft.quantization.bitsandbytes.no_peft_model", values=[True, False])

    @property
    def requires_custom_loading(self):
        return True

    @property
    def requires_augmentation(self):
        return not self._no_peft_model

    def model_loader(self, model_name, **kwargs):
        torch_dtype = kwargs.get("torch_dtype", torch.float32)
        device = kwargs.get("device")
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else "cpu"
        if torch_dtype == torch.float32 and torch.device(device).type == "cuda":
            warnings.warn("4-bit weights with fp32 compute: the fused kernels need bf16 or fp16")
        quant_type = self._quant_type

        def quantise_layer(layer):
            return quantize_linears_(
                layer, lambda lin: Linear4bit.from_linear(lin, quant_type, 64, torch_dtype))

        model = build_model(model_name, device=device, dtype=torch_dtype, layer_hook=quantise_layer)
        model.is_loaded_in_4bit = True
        model.quantization_method = "bitsandbytes"
        return model

    def augmentation(self, model, train_args, modifiable_args: Tuple):
        assert train_args.bf16 is True or train_args.fp16 is True, (
            f"{self.__class__} requires mixed precision argument `--fp16` or `--bf16`")
        (peft_config,) = modifiable_args
        assert peft_config is not None, "need peft_config to install PEFT adapters"
        model = _prepare_model_for_kbit_training(
            model, use_gradient_checkpointing=train_args.gradient_checkpointing,
            gradient_checkpointing_kwargs=train_args.gradient_checkpointing_kwargs)
        qm = getattr(model, "quantization_method", None)
        model = get_peft_model(model, peft_config)
        if qm is not None:
            model.quantization_method = qm
        return model, (None,)

    def get_callbacks_and_ready_for_train(self, model=None, accelerator=None):
        if accelerator is not None and getattr(accelerator.state, "fsdp_plugin", None) is not None and model is not None:
            plugin = accelerator.state.fsdp_plugin
            base = model if self._no_peft_model or not hasattr(model, "get_base_model") else model.get_base_model()
            plugin.param_init_fn = ensure_weights_retied(plugin.param_init_fn, base, accelerator.device)
            if model is not None and next(model.parameters()).is_cuda:
                from ...parallel.engine import install_engine

                install_engine(model, accelerator)
        return []


AccelerationPlugin.register_plugin(BNBAccelerationPlugin, configuration_and_paths=["peft.quantization.bitsandbytes"])
