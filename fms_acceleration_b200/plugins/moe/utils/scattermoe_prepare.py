"""Swap every sparse-MoE block of a model for a :class:`ScatterMoE` module, loading (the local shard of) the
expert weights.  Role of fms_acceleration_moe/utils/scattermoe_prepare.py:49-355 in the reference.

Device-mesh handling: ``ep_degree == 1`` -> no mesh; otherwise the world is arranged as
``(world // ep_degree, ep_degree)`` named ``(replicate, expert_parallel)``; experts are sharded along
``expert_parallel`` (rank ``r`` of that dimension owns experts ``[r * E/ep, (r+1) * E/ep)``) and replicated along
``replicate``; everything that is not an expert is replicated everywhere.
"""
from __future__ import annotations

import os
import warnings
from typing import Optional

import torch
import torch.distributed as dist
from torch import nn

from .scattermoe import ScatterMoE
from .scattermoe_constants import (KEY_EXPERT_PARALLEL, KEY_REPLICATE, KEY_SCATTERMOE_ROUTER,
                                   get_scattermoe_conv_spec_from_archs)
from .scattermoe_state_dict import (convert_state_dict, get_checkpoint_meta_from_sharded_safetensor,
                                    get_state_dict_from_checkpoint_metadata, load_weight_map)


def _moe_dims(moe_block: nn.Module, config):
    num_experts = getattr(config, "num_local_experts", None) or getattr(moe_block, "num_experts")
    top_k = getattr(config, "num_experts_per_tok", None) or getattr(moe_block, "top_k")
    inter = getattr(config, "moe_intermediate_size", 0) or getattr(config, "intermediate_size")
    return num_experts, top_k, inter


def _returns_router_logits(module: nn.Module) -> bool:
    """Whether the block being replaced hands back ``(hidden, router_logits)`` (transformers < 5 and the in-tree
    models) or the hidden states only (transformers >= 5 collects router logits through output recorders)."""
    if module.__class__.__module__.startswith("transformers."):
        try:
            import transformers

            return int(transformers.__version__.split(".")[0]) < 5
        except Exception:  # pragma: no cover
            return True
    return True


def build_ep_groups(world_size: int, ep_degree: int, rank: int):
    """(expert-parallel group of this rank, replicate group of this rank) or (None, None) for ep_degree 1."""
    if ep_degree == 1 or world_size == 1:
        return None, None
    ep_group = rep_group = None
    n_rep = world_size // ep_degree
    for i in range(n_rep):
        ranks = list(range(i * ep_degree, (i + 1) * ep_degree))
        g = dist.new_group(ranks)
        if rank in ranks:
            ep_group = g
    for j in range(ep_degree):
        ranks = list(range(j, world_size, ep_degree))
        g = dist.new_group(ranks)
        if rank in ranks:
            rep_group = g
    return ep_group, rep_group


def prepare_scattermoe(model: nn.Module, checkpoint_name_or_path: Optional[str] = None, rank: Optional[int] = None,
                       world_size: Optional[int] = None, ep_degree: int = 1, disable_distributed: bool = False,
                       key_rep: str = KEY_REPLICATE, key_ep: str = KEY_EXPERT_PARALLEL, device_type: str = "cuda",
                       mixed_precision: bool = False, lora_config=None, token_budget: Optional[int] = None):
    """``token_budget``: upper bound of the tokens one rank brings to one forward (per-device batch size x maximum
    sequence length); the expert-parallel buffers are sized from it once.  ``None``: taken from the first batch."""
    world_size = world_size if world_size is not None else (dist.get_world_size() if dist.is_initialized() else 1)
    rank = rank if rank is not None else (dist.get_rank() if dist.is_initialized() else 0)
    if disable_distributed and ep_degree > 1:
        raise ValueError("expert sharding can not be deferred to top-level sharding protocol if ep_degree > 1")
    assert world_size % ep_degree == 0, f"world size ({world_size}) not divisible by ep_size ({ep_degree})."
    config = model.config
    moe_cls, router_name, expert_name, _gating, sharded_ckpt = get_scattermoe_conv_spec_from_archs(config.architectures)
    ep_group, rep_group = build_ep_groups(world_size, ep_degree, rank)
    ep_rank = dist.get_rank(ep_group) if ep_group is not None else 0

    weight_map = None
    ckpt_dir = checkpoint_name_or_path if checkpoint_name_or_path and os.path.isdir(str(checkpoint_name_or_path)) else None
    if ckpt_dir is not None:
        try:
            weight_map = load_weight_map(ckpt_dir)
        except FileNotFoundError:
            weight_map = None

    swapped = []
    for name, module in list(model.named_modules()):
        if module.__class__.__name__ != moe_cls:
            continue
        parent_name, _, leaf = name.rpartition(".")
        parent = model.get_submodule(parent_name) if parent_name else model
        num_experts, top_k, inter = _moe_dims(module, config)
        assert num_experts % ep_degree == 0, f"number of moe experts ({num_experts}) not divisible by ep_size ({ep_degree})."
        per = num_experts // ep_degree
        e0, e1 = ep_rank * per, (ep_rank + 1) * per
        p0 = next(module.parameters())
        dtype, device = p0.dtype, p0.device

        if weight_map is not None and any(k.startswith(name + ".") for k in weight_map):
            meta = get_checkpoint_meta_from_sharded_safetensor(weight_map, parent_name, leaf, router_name, expert_name)
            sd = get_state_dict_from_checkpoint_metadata(ckpt_dir, meta, num_experts, inter, e0, e1, dtype)
        else:
            # convert the weights that are already in memory
            local_sd = {f"{name}.{k}": v for k, v in module.state_dict().items()}
            fake_map = {k: "<memory>" for k in local_sd}
            meta = get_checkpoint_meta_from_sharded_safetensor(fake_map, parent_name, leaf, router_name, expert_name)
            sd = convert_state_dict(name + ".", meta, local_sd, num_experts, inter, dtype)
            for k in list(sd):
                if k != KEY_SCATTERMOE_ROUTER:
                    sd[k] = sd[k][e0:e1].contiguous()

        moe = ScatterMoE(hidden_size=config.hidden_size, hidden_act=getattr(config, "hidden_act", "silu"),
                         intermediate_size=inter, num_experts=num_experts, top_k=top_k, dtype=dtype, device=device,
                         ep_group=ep_group, lora_config=lora_config, token_budget=token_budget)
        with torch.no_grad():
            moe.router.weight.copy_(sd[KEY_SCATTERMOE_ROUTER].to(device))
            for w in ("w1", "w2", "w3"):
                getattr(moe, w).weight.copy_(sd[f"{w}.weight"].to(device))
        if ep_degree > 1:
            # the loss is averaged over all ranks while every expert only lives on world/ep of them
            for w in ("w1", "w2", "w3"):
                for p in getattr(moe, w).parameters():
                    p._fmsb_expert_parallel = True
                    p._fmsb_replicate_group = rep_group
                    p._fmsb_ep_group = ep_group
        moe._fmsb_replicate_group = rep_group
        moe.return_router_logits = _returns_router_logits(module)
        setattr(parent, leaf, moe)
        swapped.append(name)
        del module
    if not swapped:
        warnings.warn(f"no '{moe_cls}' module found: nothing was converted to ScatterMoE")
    return SwappedModules(swapped)


class SwappedModules(set):
    """What :func:`prepare_scattermoe` returns: the attribute names of the replaced blocks inside their decoder layer
    (e.g. ``{"block_sparse_moe"}``, the set the reference returns, scattermoe_prepare.py:223,347,355, so that
    ``getattr(layer, name)`` finds them), with the full dotted path of every replaced module in ``paths``."""

    def __init__(self, paths):
        super().__init__(p.rpartition(".")[2] for p in paths)
        self.paths = list(paths)


def load_experts_onto_device(module: nn.Module, state_dict, device_mesh=None, num_experts_per_device: Optional[int] = None):
    """Copy router and expert weights into a ``ScatterMoE`` module (the reference's helper of this name,
    scattermoe_prepare.py:49-108, which also wraps them as DTensors).  ``state_dict`` maps ``router.weight`` /
    ``w1.weight`` ... (also the LoRA factors) to tensors that hold either all ``E`` experts or already this rank's
    ``E / ep``; a rank keeps the slice of dimension 0 that it owns.  ``device_mesh``: a process group, a DeviceMesh
    whose last dimension is the expert-parallel one, or None (the module's own group)."""
    group = device_mesh
    if device_mesh is not None and hasattr(device_mesh, "get_group"):
        group = device_mesh.get_group(device_mesh.ndim - 1)
    if group is None:
        group = getattr(module, "ep_group", None)
    rank = torch.distributed.get_rank(group) if group is not None else 0
    with torch.no_grad():
        for name, value in state_dict.items():
            path, _, leaf = name.rpartition(".")
            dst = getattr(module.get_submodule(path) if path else module, leaf)
            per = num_experts_per_device if num_experts_per_device is not None else dst.shape[0]
            if "router" not in name and value.shape[0] > per:
                value = value[rank * per:(rank + 1) * per]
            dst.copy_(value.to(device=dst.device, dtype=dst.dtype))
    return module
