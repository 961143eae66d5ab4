"""GPTQ-LoRA plugin - configuration path ``peft.quantization.auto_gptq``.

Lifecycle as in fms_acceleration_peft/framework_plugin_autogptq.py:44-395 of the reference: the loader builds
a model whose linears are GPTQ ``QuantLinear`` modules from a quantised checkpoint (``from_quantized: True`` is
the only supported mode, ``kernel`` must be ``triton_v2`` for configuration compatibility - the kernel that
actually runs is this package's CUDA dequant + tcgen05 GEMM), marks it ``is_loaded_in_4bit`` /
``quantization_method = "gptq"``, and the augmentation installs LoRA adapters and returns ``peft_config=None``.
Unlike the reference, bf16 compute is allowed in addition to fp16.
"""
from __future__ import annotations

import os
from typing import Dict, Tuple

import torch

from ...framework.framework_plugin import AccelerationPlugin
from .autogptq_utils import requires_installation_on_all_linears
from .framework_plugin_bnb import _prepare_model_for_kbit_training


def _package_available(name: str) -> bool:
    try:
        from transformers.utils import import_utils

        found = import_utils._is_package_available(name)
        return bool(found[0] if isinstance(found, tuple) else found)
    except Exception:  # transformers absent or its helper renamed
        import importlib.util

        return importlib.util.find_spec(name) is not None


class AutoGPTQAccelerationPlugin(AccelerationPlugin):
    require_packages = None

    def __init__(self, configurations: Dict[str, Dict]):
        super().__init__(configurations)
        self._check_config_equal(key="peft.quantization.auto_gptq.kernel", value="triton_v2")
        self._check_config_equal(key="peft.quantization.auto_gptq.from_quantized", value=True)
        self.use_external_lib = self._check_config_and_maybe_check_values(
            key="peft.quantization.auto_gptq.use_external_lib", values=[True, False], default=False)
        if self.use_external_lib:
            # the reference would now load through the external ``auto_gptq`` package; asking for it without having
            # it is the same error here.  When it is installed the in-tree loader and kernels are used all the same
            # (there is one GPTQ path in this package) and a warning says so.
            assert _package_available("auto_gptq"), (
                "Unable to use external library, auto_gptq module not found. "
                "Refer to README for installation instructions  as a specific version might be required.")
            import warnings

            warnings.warn("use_external_lib is set, but this package always runs its own GPTQ loader and kernels")

    @property
    def requires_custom_loading(self):
        return True

    @property
    def requires_augmentation(self):
        return True

    def model_loader(self, model_name, **kwargs):
        from .gptqmodel import GPTQModel, QuantizeConfig

        torch_dtype = kwargs.get("torch_dtype", torch.float16)
        device = kwargs.get("device")
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else "cpu"
        quantize_config = kwargs.get("quantize_config")
        is_dir = isinstance(model_name, str) and os.path.isdir(model_name)
        if quantize_config is None and not is_dir:
            # an architecture preset instead of a checkpoint: synthetic 4-bit weights, group size 128, symmetric,
            # sequential groups (the layout of the published GPTQ checkpoints the reference benchmarks)
            quantize_config = QuantizeConfig(bits=4, group_size=128, desc_act=False, sym=True)
        model = GPTQModel.from_quantized(model_name, quantize_config=quantize_config, torch_dtype=torch_dtype,
                                         device=device, low_cpu_mem_usage=kwargs.get("low_cpu_mem_usage", False))
        inner = getattr(model, "model", model)
        inner.is_loaded_in_4bit = True
        inner.quantization_method = "gptq"
        return inner

    def augmentation(self, model, train_args, modifiable_args: Tuple):
        from .gptqmodel.utils.peft import get_gptq_peft_model

        (peft_config,) = modifiable_args
        assert peft_config is not None, "need peft_config to install PEFT adapters"
        assert train_args.fp16 is True or train_args.bf16 is True, (
            f"{self.__class__} requires mixed precision argument `--fp16` or `--bf16`")
        model = _prepare_model_for_kbit_training(
            model, use_gradient_checkpointing=train_args.gradient_checkpointing,
            gradient_checkpointing_kwargs=train_args.gradient_checkpointing_kwargs)
        qm = getattr(model, "quantization_method", "gptq")
        model = get_gptq_peft_model(model, peft_config=peft_config,
                                    auto_find_all_linears=requires_installation_on_all_linears(
                                        peft_config, getattr(getattr(model, "config", None), "model_type", None)),
                                    train_mode=True)
        model.quantization_method = qm
        return model, (None,)

    def get_callbacks_and_ready_for_train(self, model=None, accelerator=None):
        if (accelerator is not None and getattr(accelerator.state, "fsdp_plugin", None) is not None
                and model is not None and next(model.parameters()).is_cuda):
            from ...parallel.engine import install_engine

            install_engine(model, accelerator)
        return []


AccelerationPlugin.register_plugin(AutoGPTQAccelerationPlugin, configuration_and_paths=["peft.quantization.auto_gptq"])
