"""Minimal LoRA layer set with PEFT-compatible attribute and state-dict names.

The fused ops of the reference read exactly these attributes from a PEFT LoRA layer
(fms_acceleration_foak/fused_ops/unsloth_lora/utils.py:66-83): ``base_layer``, ``lora_A[adapter].weight``,
``lora_B[adapter].weight``, ``scaling[adapter]``, ``lora_dropout[adapter]``, ``active_adapters``,
``disable_adapters``, ``merged``.  State-dict keys come out as
``base_model.model.<path>.lora_A.default.weight`` like PEFT's, which the checkpoint converter relies on
(fms_acceleration_moe/utils/checkpoint_utils.py:645-667).  When the real ``peft`` package is importable it
can be used instead; this module exists because the target image does not ship it.
"""
from __future__ import annotations

import json
import math
import os
import re
from dataclasses import asdict, dataclass
from typing import List, Optional, Union

import torch
from torch import nn


@dataclass
class LoraConfig:
    r: int = 8
    lora_alpha: int = 16
    lora_dropout: float = 0.0
    target_modules: Optional[Union[List[str], str]] = None
    bias: str = "none"
    task_type: str = "CAUSAL_LM"
    peft_type: str = "LORA"
    base_model_name_or_path: Optional[str] = None
    inference_mode: bool = False
    fan_in_fan_out: bool = False
    init_lora_weights: bool = True
    modules_to_save: Optional[List[str]] = None

    def to_dict(self):
        d = asdict(self)
        if isinstance(d["target_modules"], (set, tuple)):
            d["target_modules"] = sorted(d["target_modules"])
        return d


class LoraLinear(nn.Module):
    """``y = base(x) + scaling * B(A(dropout(x)))``."""

    def __init__(self, base_layer: nn.Module, r: int, lora_alpha: float, lora_dropout: float = 0.0,
                 adapter_name: str = "default", dtype=None):
        super().__init__()
        self.base_layer = base_layer
        in_f = base_layer.in_features if hasattr(base_layer, "in_features") else base_layer.infeatures
        out_f = base_layer.out_features if hasattr(base_layer, "out_features") else base_layer.outfeatures
        self.in_features, self.out_features = in_f, out_f
        dev = next((b.device for b in list(base_layer.parameters()) + list(base_layer.buffers())), None)
        if dtype is None:
            dtype = getattr(base_layer, "compute_dtype", None)
        if dtype is None:
            w = getattr(base_layer, "weight", None)
            dtype = w.dtype if (w is not None and w.dtype.is_floating_point) else torch.float32
        self.r = {adapter_name: r}
        self.lora_alpha = {adapter_name: lora_alpha}
        self.scaling = {adapter_name: lora_alpha / r}
        self.lora_dropout = nn.ModuleDict(
            {adapter_name: nn.Dropout(p=lora_dropout) if lora_dropout > 0 else nn.Identity()})
        self.lora_A = nn.ModuleDict({adapter_name: nn.Linear(in_f, r, bias=False, device=dev, dtype=dtype)})
        self.lora_B = nn.ModuleDict({adapter_name: nn.Linear(r, out_f, bias=False, device=dev, dtype=dtype)})
        nn.init.kaiming_uniform_(self.lora_A[adapter_name].weight, a=math.sqrt(5))
        nn.init.zeros_(self.lora_B[adapter_name].weight)
        self.active_adapters = [adapter_name]
        self.disable_adapters = False
        self.merged = False
        for p in base_layer.parameters():
            p.requires_grad_(False)

    @property
    def active_adapter(self):
        return self.active_adapters[0]

    @property
    def weight(self):
        return getattr(self.base_layer, "weight", None)

    @property
    def bias(self):
        return getattr(self.base_layer, "bias", None)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = self.base_layer(x)
        if self.disable_adapters or self.merged:
            return y
        for name in self.active_adapters:
            A, B = self.lora_A[name], self.lora_B[name]
            xd = self.lora_dropout[name](x).to(A.weight.dtype)
            y = y + (B(A(xd)) * self.scaling[name]).to(y.dtype)
        return y


def _all_linear(targets) -> bool:
    """``"all-linear"`` as a string or as the only entry of a list (what a command line produces)."""
    if isinstance(targets, str):
        return targets in ("all-linear", "all_linear")
    return targets is not None and len(targets) == 1 and next(iter(targets)) in ("all-linear", "all_linear")


def _matches(name: str, targets) -> bool:
    if targets is None:
        return False
    if _all_linear(targets):
        return True
    if isinstance(targets, str):
        return re.fullmatch(targets, name) is not None
    leaf = name.split(".")[-1]
    return any(leaf == t or name.endswith("." + t) or name == t for t in targets)


def _is_linear_like(m: nn.Module) -> bool:
    if isinstance(m, LoraLinear):
        return False
    return isinstance(m, nn.Linear) or (
        (hasattr(m, "in_features") or hasattr(m, "infeatures")) and hasattr(m, "forward")
        and m.__class__.__name__ in ("Linear4bit", "QuantLinear", "GPTQLinear")
    )


def inject_lora(model: nn.Module, config: LoraConfig, adapter_name: str = "default", skip=("lm_head",)) -> List[str]:
    """Wrap every targeted linear-like submodule in a :class:`LoraLinear`; returns the wrapped names."""
    wrapped = []
    for name, mod in list(model.named_modules()):
        if not _is_linear_like(mod) or not _matches(name, config.target_modules):
            continue
        if _all_linear(config.target_modules) and name.split(".")[-1] in skip:
            continue
        parent_name, _, leaf = name.rpartition(".")
        parent = model.get_submodule(parent_name) if parent_name else model
        setattr(parent, leaf, LoraLinear(mod, config.r, config.lora_alpha, config.lora_dropout, adapter_name))
        wrapped.append(name)
    return wrapped


class _BaseModelHolder(nn.Module):
    def __init__(self, model):
        super().__init__()
        self.model = model

    def forward(self, *args, **kwargs):
        return self.model(*args, **kwargs)


class PeftModelShim(nn.Module):
    """Stand-in for ``peft.PeftModel``: ``self.base_model.model`` is the wrapped model."""

    def __init__(self, model: nn.Module, peft_config: LoraConfig, adapter_name: str = "default"):
        super().__init__()
        for p in model.parameters():
            p.requires_grad_(False)
        self.targeted = inject_lora(model, peft_config, adapter_name)
        if not self.targeted:
            raise ValueError(f"no module matched target_modules={peft_config.target_modules}")
        for n, p in model.named_parameters():
            if "lora_" in n:
                p.requires_grad_(True)
        self.base_model = _BaseModelHolder(model)
        self.peft_config = {adapter_name: peft_config}
        self.active_adapter = adapter_name

    @property
    def config(self):
        return self.base_model.model.config

    def get_base_model(self):
        return self.base_model.model

    def forward(self, *args, **kwargs):
        return self.base_model(*args, **kwargs)

    def __getattr__(self, name):
        try:
            return super().__getattr__(name)
        except AttributeError:
            if name == "base_model":
                raise
            return getattr(self.base_model.model, name)

    def print_trainable_parameters(self):
        t = sum(p.numel() for p in self.parameters() if p.requires_grad)
        a = sum(p.numel() for p in self.parameters())
        print(f"trainable params: {t:,} || all params: {a:,} || trainable%: {100 * t / max(a, 1):.4f}")

    def adapter_state_dict(self):
        return {k.replace(".default", ""): v for k, v in self.state_dict().items() if "lora_" in k}

    def save_pretrained(self, out_dir: str):
        from safetensors.torch import save_file

        os.makedirs(out_dir, exist_ok=True)
        sd = {k: v.detach().cpu().contiguous() for k, v in self.adapter_state_dict().items()}
        save_file(sd, os.path.join(out_dir, "adapter_model.safetensors"), metadata={"format": "pt"})
        with open(os.path.join(out_dir, "adapter_config.json"), "w", encoding="utf-8") as fh:
            json.dump(self.peft_config[self.active_adapter].to_dict(), fh, indent=2)


    def load_adapter(self, path: str, adapter_name: Optional[str] = None) -> None:
        """Read ``adapter_model.safetensors`` (PEFT's key layout, no adapter name in the keys) from directory ``path``
        into this model's adapter tensors; every adapter tensor has to be there."""
        from safetensors.torch import load_file

        name = adapter_name or self.active_adapter
        stored = load_file(os.path.join(path, "adapter_model.safetensors"))
        own = {k.replace(f".{name}", ""): v for k, v in self.state_dict().items() if "lora_" in k}
        missing = sorted(set(own) - set(stored))
        if missing:
            raise KeyError(f"adapter file lacks {missing[:4]}{'...' if len(missing) > 4 else ''}")
        with torch.no_grad():
            for k, dst in own.items():
                dst.copy_(stored[k].to(device=dst.device, dtype=dst.dtype))

    @classmethod
    def from_pretrained(cls, model: nn.Module, path: str, adapter_name: str = "default", is_trainable: bool = False):
        """Wrap ``model`` with the adapter saved under ``path`` (``adapter_config.json`` + ``adapter_model.safetensors``,
        what :meth:`save_pretrained` and the trainer's checkpoints write)."""
        with open(os.path.join(path, "adapter_config.json"), encoding="utf-8") as fh:
            raw = json.load(fh)
        fields = LoraConfig.__dataclass_fields__
        peft = cls(model, LoraConfig(**{k: v for k, v in raw.items() if k in fields}), adapter_name)
        peft.load_adapter(path, adapter_name)
        if not is_trainable:
            for p in peft.parameters():
                p.requires_grad_(False)
        return peft

    def merge_and_unload(self) -> nn.Module:
        """Fold every adapter into its dense base weight (``W += scaling * B A``) and hand back the plain model.
        A packed 4-bit or GPTQ base cannot take the update and is refused."""
        model = self.base_model.model
        for name, mod in list(model.named_modules()):
            if not isinstance(mod, LoraLinear):
                continue
            base = mod.base_layer
            if not isinstance(base, nn.Linear):
                raise NotImplementedError(f"{name}: a LoRA adapter cannot be merged into a {type(base).__name__} base")
            ad = mod.active_adapter
            A, B = mod.lora_A[ad].weight, mod.lora_B[ad].weight
            with torch.no_grad():
                base.weight.add_((B.float() @ A.float() * mod.scaling[ad]).to(base.weight.dtype))
            parent_name, _, leaf = name.rpartition(".")
            setattr(model.get_submodule(parent_name) if parent_name else model, leaf, base)
        return model


def get_peft_model(model: nn.Module, peft_config, adapter_name: str = "default"):
    """Use ``peft.get_peft_model`` when PEFT is installed and the config is a PEFT config; otherwise the shim."""
    if not isinstance(peft_config, LoraConfig):
        try:
            import peft  # type: ignore

            return peft.get_peft_model(model, peft_config, adapter_name=adapter_name)
        except ImportError:
            pass
    return PeftModelShim(model, peft_config, adapter_name)
