"""``GPTQModel``: entry points ``from_pretrained`` (a float model to be quantised) and ``from_quantized``
(an already quantised checkpoint), dispatching on the architecture.  Role of
fms_acceleration_peft/gptqmodel/models/auto.py:36-124 in the reference."""
from __future__ import annotations

from typing import Optional

import torch

from fms_acceleration_b200.models.builder import resolve_config
from ..quantization.config import QuantizeConfig
from ..utils.backend import Backend
from .base import BaseGPTQModel
from .families import (DbrxConvertedGPTQ, DbrxGPTQ, GemmaGPTQ, GPTBigCodeGPTQ, GPTNeoXGPTQ, GraniteGPTQ, LlamaGPTQ,
                       MistralGPTQ, MixtralGPTQ)

MODEL_MAP = {
    "gpt_neox": GPTNeoXGPTQ,
    "llama": LlamaGPTQ,
    "gpt_bigcode": GPTBigCodeGPTQ,
    "mistral": MistralGPTQ,
    "mixtral": MixtralGPTQ,
    "gemma": GemmaGPTQ,
    "granite": GraniteGPTQ,
    "dbrx": DbrxGPTQ,
    "dbrx_converted": DbrxConvertedGPTQ,
}


def _model_type(model_name_or_cfg) -> str:
    cfg = resolve_config(model_name_or_cfg)
    if cfg.model_type not in MODEL_MAP:
        raise TypeError(f"{cfg.model_type} isn't supported yet.")
    return cfg.model_type


class GPTQModel:
    def __init__(self):
        raise EnvironmentError("GPTQModel is created through GPTQModel.from_pretrained / from_quantized")

    @classmethod
    def from_pretrained(cls, pretrained_model_name_or_path, quantize_config: QuantizeConfig, **model_init_kwargs) -> BaseGPTQModel:
        return MODEL_MAP[_model_type(pretrained_model_name_or_path)].from_pretrained(
            pretrained_model_name_or_path, quantize_config, **model_init_kwargs)

    @classmethod
    def from_quantized(cls, model_name_or_path, quantize_config: Optional[QuantizeConfig] = None,
                       backend: Backend = Backend.AUTO, torch_dtype=torch.float16, device=None, **kwargs) -> BaseGPTQModel:
        return MODEL_MAP[_model_type(model_name_or_path)].from_quantized(
            model_name_or_path, quantize_config=quantize_config, backend=backend, torch_dtype=torch_dtype,
            device=device, **kwargs)
