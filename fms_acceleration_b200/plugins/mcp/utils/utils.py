"""Install context parallelism on the Mamba2 layers of a model.

Role of fms_acceleration_mcp/utils/utils.py:34-140 in the reference: build the mesh ``(cp,)`` or
``(world // cp, cp)`` named ``("dp_shard", "cp")``, and give every ``layer.mamba`` of ``model.model.layers`` a
context-parallel scan while keeping its parameters (and therefore the checkpoint format) unchanged.  The reference
swaps in the external ``mamba_ssm`` ``Mamba2CP`` module; here the in-tree mixer keeps its weights and receives a
:class:`ContextParallel` communicator (``parallel/context_parallel.py``).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch.distributed as dist

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
    inner = getattr(base, "model", base)
    patched = 0
    for layer in inner.layers:
        mixer = getattr(layer, "mamba", None)
        if mixer is None:
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
