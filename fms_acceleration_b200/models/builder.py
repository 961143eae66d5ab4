"""Model construction helpers: random-init models of a preset architecture, quantised layer by layer."""
from __future__ import annotations

import contextlib
import json
import os
import re
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


class _CheckpointReader:
    """Tensors of a local safetensors checkpoint (one file, or shards with ``model.safetensors.index.json``), read one
    at a time."""

    _LAYER = re.compile(r"^(?:.*\.)?(?:layers|h)\.(\d+)\.(.+)$")

    def __init__(self, directory: str):
        self.directory = directory
        index = os.path.join(directory, "model.safetensors.index.json")
        single = os.path.join(directory, "model.safetensors")
        if os.path.exists(index):
            with open(index, encoding="utf-8") as fh:
                self.weight_map = dict(json.load(fh)["weight_map"])
        elif os.path.exists(single):
            from safetensors import safe_open

            with safe_open(single, framework="pt") as f:
                self.weight_map = {k: "model.safetensors" for k in f.keys()}
        else:
            self.weight_map = {}
        self.by_layer = {}
        for key in self.weight_map:
            m = self._LAYER.match(key)
            if m:
                self.by_layer.setdefault(int(m.group(1)), {})[m.group(2)] = key
        self._open = {}

    def __bool__(self):
        return bool(self.weight_map)

    def tensor(self, key: str) -> torch.Tensor:
        from safetensors import safe_open

        name = self.weight_map[key]
        if name not in self._open:
            self._open[name] = safe_open(os.path.join(self.directory, name), framework="pt")
        return self._open[name].get_tensor(key)

    def load_layer(self, layer: nn.Module, index: int) -> None:
        """Copy the tensors stored for decoder layer ``index`` into ``layer`` (names relative to the layer)."""
        own = dict(layer.named_parameters())
        own.update(dict(layer.named_buffers()))
        with torch.no_grad():
            for rest, key in self.by_layer.get(index, {}).items():
                if rest in own:
                    own[rest].copy_(self.tensor(key).to(own[rest].dtype))

    def load_rest(self, model: nn.Module) -> None:
        """Everything that does not belong to a decoder layer (embeddings, final norm, output head)."""
        layer_keys = {k for d in self.by_layer.values() for k in d.values()}
        own = dict(model.named_parameters())
        own.update(dict(model.named_buffers()))
        with torch.no_grad():
            for key in self.weight_map:
                if key not in layer_keys and key in own:
                    own[key].copy_(self.tensor(key).to(own[key].dtype))


def build_model(model_name_or_cfg, device="cpu", dtype=torch.float32, layer_hook: Optional[Callable] = None,
                seed: Optional[int] = None) -> nn.Module:
    """A model built directly on ``device``: random-init (normal(0, initializer_range)) for a preset, with the weights of
    the checkpoint for a local directory that holds safetensors files.  ``layer_hook`` runs on every decoder layer
    right after its construction, and after that layer's checkpoint tensors are in place (so a hook that quantises
    the layer packs the real weights, one layer at a time)."""
    cfg = resolve_config(model_name_or_cfg)
    cls = _registry()[cfg.architectures[0]]
    if seed is not None:
        torch.manual_seed(seed)
    reader = _CheckpointReader(cfg.name_or_path) if cfg.name_or_path and os.path.isdir(cfg.name_or_path) else None
    hook = layer_hook
    if reader and layer_hook is not None:
        seen = [0]

        def hook(layer):  # noqa: F811 - decoder layers are constructed in order
            reader.load_layer(layer, seen[0])
            seen[0] += 1
            return layer_hook(layer)

    with torch.device(device), _default_dtype(dtype):
        model = cls(cfg, layer_hook=hook)
    if reader:
        if layer_hook is None:
            state = {k: reader.tensor(k) for k in reader.weight_map}
            model.load_state_dict(state, strict=False)
        else:
            reader.load_rest(model)
    return model


def quantize_linears_(module: nn.Module, make_quant: Callable[[nn.Linear], nn.Module], skip=("lm_head",)) -> nn.Module:
    """Replace every ``nn.Linear`` below ``module`` (except ``skip``) by ``make_quant(linear)``."""
    for name, child in list(module.named_children()):
        if isinstance(child, nn.Linear) and name not in skip:
            setattr(module, name, make_quant(child))
        else:
            quantize_linears_(child, make_quant, skip)
    return module
