"""Model construction helpers: random-init models of a preset architecture, quantised layer by layer."""
from __future__ import annotations

import contextlib
import json
import os
from typing import Callable, Optional

import torch
from torch import nn

from .config import HUB_ALIASES, PRESETS, DecoderConfig, preset

ARCH_TO_MODEL = {}


def _registry():
    if not ARCH_TO_MODEL:
        from .llama import GraniteForCausalLM, LlamaForCausalLM, MistralForCausalLM

        ARCH_TO_MODEL.update({
            "LlamaForCausalLM": LlamaForCausalLM,
            "MistralForCausalLM": MistralForCausalLM,
            "GraniteForCausalLM": GraniteForCausalLM,
        })
        try:
            from .granitemoe import GraniteMoeForCausalLM

            ARCH_TO_MODEL["GraniteMoeForCausalLM"] = GraniteMoeForCausalLM
        except ImportError:
            pass
        from .gpt_bigcode import GPTBigCodeForCausalLM
        from .granitemoe import GraniteMoeSharedForCausalLM
        from .mixtral import MixtralForCausalLM

        ARCH_TO_MODEL.update({"MixtralForCausalLM": MixtralForCausalLM,
                              "GraniteMoeSharedForCausalLM": GraniteMoeSharedForCausalLM,
                              "GPTBigCodeForCausalLM": GPTBigCodeForCausalLM})
        try:
            from .granitemoehybrid import GraniteMoeHybridForCausalLM

            ARCH_TO_MODEL["GraniteMoeHybridForCausalLM"] = GraniteMoeHybridForCausalLM
        except ImportError:
            pass
        try:
            from .mamba2 import Mamba2ForCausalLM

            ARCH_TO_MODEL["Mamba2ForCausalLM"] = Mamba2ForCausalLM
        except ImportError:
            pass
    return ARCH_TO_MODEL


def resolve_config(model_name_or_cfg) -> DecoderConfig:
    """A preset name, a directory holding ``config.json`` or a ready ``DecoderConfig``."""
    if isinstance(model_name_or_cfg, DecoderConfig):
        return model_name_or_cfg
    name = str(model_name_or_cfg)
    if name in PRESETS or name in HUB_ALIASES:
        cfg = preset(name)
        cfg.name_or_path = name
        return cfg
    cfg_file = os.path.join(name, "config.json")
    if os.path.exists(cfg_file):
        with open(cfg_file, encoding="utf-8") as fh:
            raw = json.load(fh)
        fields = DecoderConfig.__dataclass_fields__
        cfg = DecoderConfig(**{k: v for k, v in raw.items() if k in fields})
        cfg.name_or_path = name
        return cfg
    raise ValueError(f"unknown model {name!r}: not a preset ({sorted(PRESETS)}) and no config.json there")


@contextlib.contextmanager
def _default_dtype(dtype):
    old = torch.get_default_dtype()
    torch.set_default_dtype(dtype)
    try:
        yield
    finally:
        torch.set_default_dtype(old)


def build_model(model_name_or_cfg, device="cpu", dtype=torch.float32, layer_hook: Optional[Callable] = None,
                seed: Optional[int] = None) -> nn.Module:
    """Random-init model (normal(0, initializer_range)), built directly on ``device``; ``layer_hook`` runs on
    every decoder layer right after its construction."""
    cfg = resolve_config(model_name_or_cfg)
    cls = _registry()[cfg.architectures[0]]
    if seed is not None:
        torch.manual_seed(seed)
    with torch.device(device), _default_dtype(dtype):
        model = cls(cfg, layer_hook=layer_hook)
    state_file = os.path.join(cfg.name_or_path, "model.safetensors") if cfg.name_or_path else ""
    if state_file and os.path.exists(state_file) and layer_hook is None:
        from safetensors.torch import load_file

        model.load_state_dict(load_file(state_file), strict=False)
    return model


def quantize_linears_(module: nn.Module, make_quant: Callable[[nn.Linear], nn.Module], skip=("lm_head",)) -> nn.Module:
    """Replace every ``nn.Linear`` below ``module`` (except ``skip``) by ``make_quant(linear)``."""
    for name, child in list(module.named_children()):
        if isinstance(child, nn.Linear) and name not in skip:
            setattr(module, name, make_quant(child))
        else:
            quantize_linears_(child, make_quant, skip)
    return module
