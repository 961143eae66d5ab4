"""Builders of fused LoRA forwards for module-by-module patching of Hugging Face attention / MLP modules
(role of fms_acceleration_foak/models/utils.py:31-224 in the reference).

The fused op for ``q_proj``/``k_proj``/``v_proj`` runs when the FIRST of the three projections is called and
caches the other two results; the following two calls return the cached tensors.  This keeps the attention
module's own forward untouched.
"""
from __future__ import annotations

from typing import Callable, List, Tuple

import torch

from ....framework.model_patcher import ModelPatcherTrigger
from ....ops.fused_layer import _scaled  # noqa: F401
from ....ops.proj import ProjGroup


def _is_lora_layer(m: torch.nn.Module) -> bool:
    return hasattr(m, "lora_A") and hasattr(m, "lora_B") and hasattr(m, "base_layer")


def trigger_fused_ops(module: torch.nn.Module, attn_cls, submodule_names: List[str]) -> bool:
    """Fires on instances of ``attn_cls`` all of whose named submodules carry LoRA adapters."""
    if not isinstance(module, attn_cls):
        return False
    return all(_is_lora_layer(getattr(module, n, None)) for n in submodule_names if hasattr(module, n)) and \
        all(hasattr(module, n) for n in submodule_names)


class _GroupFn(torch.autograd.Function):
    """Autograd wrapper of ``ProjGroup.forward/backward`` for a flattened input."""

    @staticmethod
    def forward(ctx, x2, group: ProjGroup, *params):
        aux = {}  # receives the keep mask when the adapters have input dropout
        y, xa = group.forward(x2, aux=aux)
        ctx.group, ctx.aux = group, aux
        ctx.save_for_backward(x2, xa)
        return y

    @staticmethod
    def backward(ctx, dy):
        x2, xa = ctx.saved_tensors
        dx, grads = ctx.group.backward(dy.contiguous(), x2, xa, need_dx=ctx.needs_input_grad[0], aux=ctx.aux)
        return (dx, None, *grads)


def _group_bias(group: ProjGroup, dtype, device):
    """The biases of the group's base layers side by side (zeros for a layer without one), or None when no layer has
    a bias.  Added after the fused product, as the reference's fused functions do
    (fused_ops/unsloth_lora/bnb/fast_lora.py:72-76); a bias that is trained takes its gradient through this sum."""
    biases = [getattr(b, "bias", None) for b in group.bases]
    if all(b is None for b in biases):
        return None
    parts = [b.to(dtype) if b is not None else torch.zeros(n, dtype=dtype, device=device)
             for b, n in zip(biases, group.out_sizes)]
    return parts[0] if len(parts) == 1 else torch.cat(parts)


def _run_group(group: ProjGroup, x: torch.Tensor) -> torch.Tensor:
    x2 = x.reshape(-1, x.shape[-1])
    if x2.stride(1) != 1 or x2.stride(0) % 8:
        x2 = x2.contiguous()
    y = _GroupFn.apply(x2, group, *group.trainable())
    bias = _group_bias(group, y.dtype, y.device)
    if bias is not None:
        y = y + bias
    return y.view(*x.shape[:-1], y.shape[-1])


def build_lora_fused_ops(attn: torch.nn.Module, base_type: str = "auto_gptq", submodule_names=None,
                         fused_op: str = "qkv") -> List[Tuple[ModelPatcherTrigger, Callable]]:
    """Returns ``[(trigger, forward), ...]`` for the named submodules of ``attn`` (nested, isolated patch)."""
    names = list(submodule_names)
    mods = [getattr(attn, n) for n in names]
    if fused_op == "mlp":
        # order the group as gate | up, down separately
        gate, up, down = attn.gate_proj, attn.up_proj, attn.down_proj
        gu = ProjGroup([gate, up], f"hf.{id(attn)}.gate_up")
        dn = ProjGroup([down], f"hf.{id(attn)}.down")
        inter = gu.out_sizes[0]

        def mlp_forward(self, x):
            from ....ops.activation import glu

            y = _run_group(gu, x)
            h = glu(y[..., :inter], y[..., inter:], "silu")
            return _run_group(dn, h)

        # the MLP module itself gets the fused forward: signalled by returning a plain callable
        return mlp_forward

    group = ProjGroup(mods, f"hf.{id(attn)}.{fused_op}")
    cache = {}

    def make_forward(idx: int, name: str):
        def _forward(self, x):
            key = (x.data_ptr(), x._version, tuple(x.shape))
            if cache.get("key") != key or name not in cache.get("left", ()):
                y = _run_group(group, x)
                outs = torch.split(y, group.out_sizes, dim=-1)
                cache["key"] = key
                cache["outs"] = outs
                cache["left"] = set(names)
            cache["left"].discard(name)
            out = cache["outs"][idx]
            if not cache["left"]:
                cache.pop("outs", None)
                cache["key"] = None
            return out

        return _forward

    return [(ModelPatcherTrigger(check=(lambda m, _t=mod: m is _t), module_name=n), make_forward(i, n))
            for i, (n, mod) in enumerate(zip(names, mods))]


KEY_HIDDEN_ACTIVATIONS = ["hidden_act", "activation_function"]


def get_hidden_activation_fn_key(config) -> str:
    """The MLP activation named by a model configuration, read from ``hidden_act`` (most families) or
    ``activation_function`` (GPTBigCode); fms_acceleration_foak/models/utils.py:208-217."""
    for key in KEY_HIDDEN_ACTIVATIONS:
        value = getattr(config, key, None)
        if value:
            return value
    raise ValueError(f"Unable to determine activation function key for architecture {getattr(config, 'architectures', None)}.")


def get_transformers_version():
    """Installed ``transformers`` version string, or None."""
    try:
        from importlib.metadata import version

        return version("transformers")
    except Exception:  # noqa: BLE001 - not installed
        return None
