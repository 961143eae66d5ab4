"""Helpers around GPTQ layers and LoRA installation (the reference's fms_acceleration_peft/autogptq_utils.py:34-216).

Two groups:

* deciding whether adapters go on every linear (``requires_installation_on_all_linears``) and building / placing the
  LoRA module for a quantised layer (``create_new_module_peft``, ``replace_module_peft``);
* the float-view trick for sharding wrappers that only flatten floating-point parameters: the packed int32
  ``qweight`` / ``qzeros`` buffers are re-registered as frozen ``nn.Parameter`` views in a float dtype and the layer's
  forward views them back as int32 just before it runs.  This package's own sharded engine keeps the packed tensors
  as they are (it shards bytes, ``parallel/engine.py``), so the trick is only needed under an external wrapper.
"""
from __future__ import annotations

from functools import partial
from typing import Callable, List, Optional, Union

import torch

from ...framework.model_patcher import ModelPatcher, ModelPatcherRule, ModelPatcherTrigger

# the packed tensors of a GPTQ layer that a float-only sharding wrapper cannot flatten as they are
PATCH_FOR_FSDP_TRITON_V2 = ["qweight", "qzeros"]
PEFT_ALL_LINEAR = "all-linear"

# per model type, where adapters go when the LoRA config names no target modules
_DEFAULT_TARGETS = {
    "llama": ["q_proj", "v_proj"], "mistral": ["q_proj", "v_proj"], "mixtral": ["q_proj", "v_proj"],
    "granite": ["q_proj", "v_proj"], "gemma": ["q_proj", "v_proj"], "gpt_bigcode": ["c_attn"],
    "gpt_neox": ["query_key_value"],
}


def requires_installation_on_all_linears(peft_config, model_type: Optional[str] = None) -> bool:
    """True when ``target_modules`` is the ``all-linear`` wildcard (alone).  With no target modules the defaults of
    ``model_type`` are looked up (peft's table when peft is installed, else the in-tree one) and an unknown type is
    an error."""
    tm = getattr(peft_config, "target_modules", None)
    if tm is None:
        try:
            from peft.utils.constants import TRANSFORMERS_MODELS_TO_LORA_TARGET_MODULES_MAPPING as table  # type: ignore
        except ImportError:
            table = _DEFAULT_TARGETS
        if model_type not in table:
            raise ValueError("target modules not specified and unable to determine default "
                             f"for given model type {model_type}.")
        tm = table[model_type]
    if not isinstance(tm, (list, set, tuple, str)):
        raise TypeError("if provided, target modules can only be list, set or string")
    if isinstance(tm, str):
        return tm in (PEFT_ALL_LINEAR, "all_linear")
    if PEFT_ALL_LINEAR not in tm:
        return False
    if len(tm) != 1:
        raise ValueError(f"`{PEFT_ALL_LINEAR}` must exist alone in target modules")
    return True


def patch_forward_to_view_attributes_before_call(old_forward: Callable, attribute_names: List[str],
                                                 torch_dtype: torch.dtype,
                                                 submodule_names: Union[str, List[str], None] = None,
                                                 is_method_forward: bool = True) -> Callable:
    """A forward that first re-views ``attribute_names`` of the module (or of the named submodules) as
    ``torch_dtype`` (a no-op when they already have it) and then calls ``old_forward`` (bound when
    ``is_method_forward``)."""
    names = [submodule_names or ""] if isinstance(submodule_names, (str, type(None))) else list(submodule_names)

    def _forward(self, *args, **kwargs):
        for sub in names:
            mod = self.get_submodule(sub)
            for attr_name in attribute_names:
                viewed = getattr(mod, attr_name).view(torch_dtype)
                try:
                    setattr(mod, attr_name, viewed)
                except TypeError:
                    # the name is registered as a Parameter: shadow it with the plain view for this call
                    mod.__dict__[attr_name] = viewed
        if is_method_forward:
            return old_forward(*args, **kwargs)
        return old_forward(self, *args, **kwargs)

    return _forward


def build_patch_to_view_tensor_to_parameter_for_fsdp_gptq(module: torch.nn.Module, torch_dtype: torch.dtype) -> Callable:
    """Turn the packed tensors of ``module`` into frozen Parameters viewed as ``torch_dtype`` and return the forward
    that views them back as int32."""
    for name in PATCH_FOR_FSDP_TRITON_V2:
        packed = getattr(module, name)
        module._buffers.pop(name, None)
        setattr(module, name, torch.nn.Parameter(packed.view(torch_dtype), requires_grad=False))
    return patch_forward_to_view_attributes_before_call(module.forward, attribute_names=PATCH_FOR_FSDP_TRITON_V2,
                                                        torch_dtype=torch.int32)


def register_tensors_as_parameters_patch_rule(target_module, torch_dtype: torch.dtype) -> None:
    """Register the model-patcher rule that applies the float-view trick to every ``target_module`` instance."""
    ModelPatcher.register(ModelPatcherRule(
        rule_id="autogptq_patch_tensors_as_float_parameters",
        trigger=ModelPatcherTrigger(check=target_module),
        forward_builder=partial(build_patch_to_view_tensor_to_parameter_for_fsdp_gptq, torch_dtype=torch_dtype)))


def make_sure_no_tensor_in_meta_device(model: torch.nn.Module, use_triton: bool = True, desc_act: bool = False,
                                       group_size: int = 128, bits: int = 4, disable_exllama: bool = True,
                                       disable_exllamav2: bool = True, use_marlin: bool = False,
                                       use_tritonv2: bool = True) -> None:
    """Give every quantised layer whose bias was left on the meta device by a low-memory load a real zero bias on the
    CPU (the kernel-selection flags are accepted for call compatibility: there is one QuantLinear here)."""
    from .gptqmodel.nn_modules.qlinear.qlinear_tritonv2 import QuantLinear

    for m in model.modules():
        bias = getattr(m, "bias", None)
        if isinstance(m, QuantLinear) and bias is not None and bias.device.type == "meta":
            m._buffers.pop("bias", None)
            m._parameters.pop("bias", None)
            m.register_buffer("bias", torch.zeros(m.outfeatures, dtype=torch.float16, device="cpu"))


def replace_module_peft(self, parent_module, child_name, new_module, old_module) -> None:
    """Put the LoRA-wrapped layer in place of the old one and move its adapter tensors to the old layer's device."""
    setattr(parent_module, child_name, new_module)
    where = next(iter(list(old_module.parameters()) + list(old_module.buffers()))).device
    for name, module in new_module.named_modules():
        if "lora_" in name:
            module.to(where)


def create_new_module_peft(lora_config, adapter_name: str, target: torch.nn.Module, target_cls, **kwargs):
    """The LoRA module for ``target`` when it is a ``target_cls`` layer, else None (the caller then reports an
    unsupported layer)."""
    from .gptqmodel.utils.peft import GPTQLoraLinear

    if not isinstance(target, target_cls):
        return None
    return GPTQLoraLinear(target, r=kwargs.get("r", lora_config.r), lora_alpha=kwargs.get("lora_alpha", lora_config.lora_alpha),
                          lora_dropout=kwargs.get("lora_dropout", getattr(lora_config, "lora_dropout", 0.0)),
                          adapter_name=adapter_name, dtype=kwargs.get("dtype"))
