"""Install context parallelism on the Mamba2 layers of a model.

Role of fms_acceleration_mcp/utils/utils.py:34-140 in the reference: build the mesh ``(cp,)`` or
``(world // cp, cp)`` named ``("dp_shard", "cp")``, and give every ``layer.mamba`` of ``model.model.layers`` a
context-parallel scan while keeping its parameters (and therefore the checkpoint format) unchanged.  The reference
swaps in the external ``mamba_ssm`` ``Mamba2CP`` module; here the in-tree mixer keeps its weights and receives a
:class:`ContextParallel` communicator (``parallel/context_parallel.py``).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch
import torch.distributed as dist
from torch import nn

KEY_DP, KEY_CP = "dp_shard", "cp"


def hf_config_ssm_config(hf_config) -> Dict:
    """The SSM hyper-parameters of a Hugging Face style config (d_state is fixed at 128 like the reference does)."""
    return {
        "d_model": hf_config.hidden_size,
        "d_state": getattr(hf_config, "mamba_d_state", 128),
        "ngroups": getattr(hf_config, "mamba_n_groups", 1),
        "rmsnorm": True,
        "chunk_size": getattr(hf_config, "mamba_chunk_size", 256),
        "conv_bias": getattr(hf_config, "mamba_conv_bias", True),
        "d_conv": getattr(hf_config, "mamba_d_conv", 4),
    }


# the name this helper carries in the reference (fms_acceleration_mcp/utils/utils.py:51-60)
get_ssmconfig_from_hfconfig = hf_config_ssm_config


def __getattr__(name: str):
    # ``Mamba2CPHF`` is the reference's name for the module that sits behind a Hugging Face Mamba layer's call
    # convention (fms_acceleration_mcp/utils/utils.py:64-80); here that is the adapter class, made on first use
    if name == "Mamba2CPHF":
        return _adapter_class()
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


def _adapter_class():
    """``HFMamba2Adapter`` is a subclass of the in-tree mixer (so parameter names, and with them checkpoints, are
    those of the Hugging Face module); the class is made on first use to keep this module importable without the
    model zoo."""
    global _ADAPTER
    if _ADAPTER is not None:
        return _ADAPTER
    from ....models.config import DecoderConfig
    from ....models.mamba2 import Mamba2Mixer

    class HFMamba2Adapter(Mamba2Mixer):
        """The in-tree Mamba2 mixer behind the call convention of a Hugging Face Mamba2 layer.

        Built from a ``transformers`` mixer (``Mamba2Mixer``, ``GraniteMoeHybridMambaLayer``, ``BambaMixer``: same
        parameter names and projection layout) whose state dict it loads unchanged; ``forward(hidden_states
        [B, S, H], ...)`` ignores cache, mask and sequence-index arguments like the reference's ``Mamba2CPHF``
        (fms_acceleration_mcp/utils/utils.py:64-80) and runs every row of the batch as one sequence."""

        def __init__(self, hf_mixer: nn.Module, layer_idx: int = 0, eps: Optional[float] = None):
            hidden = hf_mixer.in_proj.in_features
            d_inner = hf_mixer.intermediate_size
            if d_inner % hidden != 0:
                raise ValueError("the inner width must be a multiple of the hidden size")
            if hf_mixer.n_groups != 1 and getattr(hf_mixer.norm, "group_size", d_inner) != d_inner:
                raise NotImplementedError("grouped gated RMSNorm (n_groups > 1) is not supported")
            lim = tuple(getattr(hf_mixer, "time_step_limit", (0.0, float("inf"))))
            if lim[0] > 0.0 or lim[1] != float("inf"):
                raise NotImplementedError("a time-step clamp is not supported")
            cfg = DecoderConfig(
                hidden_size=hidden, mamba_expand=d_inner // hidden, mamba_d_head=hf_mixer.head_dim,
                mamba_d_state=hf_mixer.ssm_state_size, mamba_n_groups=hf_mixer.n_groups,
                mamba_d_conv=hf_mixer.conv_kernel_size, mamba_chunk_size=hf_mixer.chunk_size,
                mamba_conv_bias=hf_mixer.conv1d.bias is not None, mamba_proj_bias=hf_mixer.in_proj.bias is not None,
                rms_norm_eps=eps if eps is not None else getattr(hf_mixer.norm, "variance_epsilon", 1e-5))
            super().__init__(cfg, layer_idx)
            self.to(device=hf_mixer.in_proj.weight.device, dtype=hf_mixer.in_proj.weight.dtype)
            self.load_state_dict(hf_mixer.state_dict())
            # per-head parameters stay in the precision the source module keeps them in
            for name in ("A_log", "D", "dt_bias"):
                getattr(self, name).data = getattr(hf_mixer, name).data.clone()

        def forward(self, hidden_states, *args, **kwargs):  # noqa: D401  (Hugging Face call convention)
            if hidden_states.dim() == 2:
                return super().forward(hidden_states)
            return torch.stack([super(HFMamba2Adapter, self).forward(row) for row in hidden_states], 0)

    _ADAPTER = HFMamba2Adapter
    return _ADAPTER


_ADAPTER = None


def _is_hf_mamba_module(m: nn.Module) -> bool:
    return all(hasattr(m, a) for a in ("in_proj", "conv1d", "A_log", "dt_bias", "out_proj", "ssm_state_size"))


def swap_hf_mamba_modules(model, names=("mamba", "mixer")) -> int:
    """Replace every Hugging Face Mamba2 layer found under one of ``names`` on a decoder layer by an
    ``HFMamba2Adapter`` (a subclass of the in-tree mixer, see :func:`_adapter_class`) with the same weights; returns how many were replaced."""
    from ....models.mamba2 import Mamba2Mixer

    adapter = _adapter_class()
    n = 0
    for parent in list(model.modules()):
        for name in names:
            child = getattr(parent, name, None)
            if isinstance(child, nn.Module) and not isinstance(child, Mamba2Mixer) and _is_hf_mamba_module(child):
                setattr(parent, name, adapter(child, layer_idx=getattr(child, "layer_idx", n)))
                n += 1
    return n


def build_cp_group(world_size: int, cp_degree: int, rank: int):
    """Consecutive ranks form one context-parallel group (the ``cp`` dimension varies fastest)."""
    if cp_degree == world_size:
        return dist.group.WORLD
    mine = None
    for i in range(world_size // cp_degree):
        ranks = list(range(i * cp_degree, (i + 1) * cp_degree))
        g = dist.new_group(ranks)
        if rank in ranks:
            mine = g
    return mine


def patch_mamba_layers_with_cp_head(model, checkpoint_name_or_path: Optional[str] = None, rank: int = 0,
                                    cp_degree: int = 2, world_size: int = 1, cp_mamba_impl: str = "allgather",
                                    cp_mamba_recompute: bool = False):
    if cp_degree == 1:
        raise ValueError("CP degree can't be one")
    if world_size % cp_degree != 0:
        raise ValueError(f"world size {world_size} is not divisible by the context-parallel degree {cp_degree}")
    if cp_mamba_impl not in ("allgather", "serial"):
        raise ValueError(f"unknown mamba_impl {cp_mamba_impl!r}")
    from ....parallel.context_parallel import ContextParallel

    group = build_cp_group(world_size, cp_degree, dist.get_rank() if dist.is_initialized() else rank)
    device = next(model.parameters()).device
    cp = ContextParallel(group, device, impl=cp_mamba_impl, recompute=cp_mamba_recompute)
    base = model.get_base_model() if hasattr(model, "get_base_model") else model
    swap_hf_mamba_modules(base, names=("mamba",))  # Hugging Face layers become the in-tree mixer, same weights
    inner = getattr(base, "model", base)
    patched = 0
    from ....models.granitemoehybrid import GraniteMoeHybridDecoderLayer

    for layer in inner.layers:
        mixer = getattr(layer, "mamba", None)
        if mixer is None:
            if getattr(layer, "self_attn", None) is not None:
                # an attention layer of a hybrid model: it has to see the keys of the earlier slices
                if not isinstance(layer, GraniteMoeHybridDecoderLayer):
                    raise NotImplementedError(
                        "context parallelism over the attention layers of a Hugging Face hybrid model: build the model "
                        "with fms_acceleration_b200.models (its attention layers gather keys and values over the group)")
                layer.cp = cp
            continue
        mixer.cp = cp
        patched += 1
    if patched == 0:
        raise ValueError("the model has no `layer.mamba` modules to run context-parallel")
    base.cp = cp
    # parameters are replicated over the context-parallel group: their gradients are summed over it
    for p in model.parameters():
        p._fmsb_cp_group = group
    return cp
