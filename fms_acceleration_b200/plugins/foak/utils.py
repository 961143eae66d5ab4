"""Helpers of the fused-ops plugin: patch-rule filtering and gradient synchronisation of LoRA adapters that
live outside the sharded-parameter engine (role of fms_acceleration_foak/utils.py:27-96 in the reference)."""
from __future__ import annotations

from typing import List, Set

import torch
import torch.distributed as dist

from ...framework.model_patcher import ModelPatcherRule


def filter_mp_rules(rules: List[ModelPatcherRule], filter_endswith: Set[str], drop: bool = False) -> List[ModelPatcherRule]:
    """Keep (or, with ``drop``, remove) the rules whose id ends with one of ``filter_endswith``."""
    hit = lambda r: any(r.rule_id.endswith(x) for x in filter_endswith)  # noqa: E731
    return [r for r in rules if (not hit(r) if drop else hit(r))]


def lora_adapters_switch_ddp_from_fsdp(modules: List[torch.nn.Module], fsdp_plugin) -> None:
    """The fused ops read ``lora_A`` / ``lora_B`` weights directly and never call the adapters' ``forward``, so
    a sharding engine that unshards parameters in ``forward`` hooks would never gather them.  Exclude the
    adapters from sharding (replicate them, broadcast from rank 0) and average their gradients across ranks.

    The reference registers one ``all_reduce`` hook per adapter tensor (utils.py:39-43, 256 small collectives
    per step for a 7B model); here the adapters are only *marked* and the engine reduces all of them in one
    fused bucket after backward (see ``parallel.grad_sync``).
    """
    ignored = list(fsdp_plugin.ignored_modules or [])
    world = dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1
    for mod in modules:
        for sub_name in ("lora_A", "lora_B"):
            sub = getattr(mod, sub_name, None)
            if sub is None:
                continue
            ignored.append(sub)
            for p in sub.parameters():
                p._fmsb_replicated = True
                if world > 1:
                    dist.broadcast(p.data, src=0)
    fsdp_plugin.ignored_modules = ignored
