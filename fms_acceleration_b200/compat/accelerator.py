"""A small ``Accelerator`` with the attributes the plugins use: ``prepare``, ``is_main_process``, ``device``,
``num_processes``, ``process_index``, ``state.fsdp_plugin``, ``reduce``, ``wait_for_everyone``.

The reference receives an ``accelerate.Accelerator`` from HF Trainer; its plugins read and mutate the FSDP
plugin object hanging off ``accelerator.state`` (``ignored_modules``, ``param_init_fn``, ``state_dict_type``;
e.g. fms_acceleration_foak/utils.py:27-80, fms_acceleration_moe/framework_plugin_scattermoe.py:113-174).  Here
the same fields configure this package's own sharded-parameter engine.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Callable, List, Optional

import torch
import torch.distributed as dist


@dataclass
class FSDPPluginShim:
    ignored_modules: Optional[List[torch.nn.Module]] = None
    param_init_fn: Optional[Callable] = None
    state_dict_type: str = "SHARDED_STATE_DICT"
    fsdp_version: int = 1
    cpu_ram_efficient_loading: bool = False
    sync_module_states: bool = True

    def set_state_dict_type(self, t: str) -> None:
        self.state_dict_type = t


@dataclass
class AcceleratorState:
    fsdp_plugin: Optional[FSDPPluginShim] = None
    distributed_type: str = "NO"
    mixed_precision: str = "no"


class Accelerator:
    def __init__(self, device=None, fsdp: Optional[bool] = None, dispatch_batches: Optional[bool] = None):
        self.num_processes = dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1
        self.process_index = dist.get_rank() if self.num_processes > 1 else 0
        self.local_process_index = int(os.environ.get("LOCAL_RANK", "0"))
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        self.device = torch.device(device)
        use_fsdp = fsdp if fsdp is not None else (
            self.num_processes > 1 or os.environ.get("ACCELERATE_USE_FSDP", "false").lower() == "true")
        self.state = AcceleratorState(
            fsdp_plugin=FSDPPluginShim() if use_fsdp else None,
            distributed_type="FSDP" if use_fsdp else ("MULTI_GPU" if self.num_processes > 1 else "NO"),
        )
        self.engine = None  # set by plugins that install a sharded-parameter engine

    @property
    def is_main_process(self) -> bool:
        return self.process_index == 0

    @property
    def is_local_main_process(self) -> bool:
        return self.local_process_index == 0

    def prepare(self, *args, device_placement=None):
        """Models are moved to the device; data loaders and everything else pass through unchanged."""
        out = []
        for a in args:
            if isinstance(a, torch.nn.Module):
                out.append(a.to(self.device) if not any(p.is_meta for p in a.parameters()) else a)
            else:
                out.append(a)
        return out[0] if len(out) == 1 else tuple(out)

    def reduce(self, tensor: torch.Tensor, reduction: str = "sum") -> torch.Tensor:
        if self.num_processes > 1:
            t = tensor.clone()
            dist.all_reduce(t, op=dist.ReduceOp.SUM)
            if reduction == "mean":
                t = t / self.num_processes
            return t
        return tensor

    def gather(self, tensor: torch.Tensor) -> torch.Tensor:
        if self.num_processes > 1:
            outs = [torch.empty_like(tensor) for _ in range(self.num_processes)]
            dist.all_gather(outs, tensor)
            return torch.cat(outs, dim=0)
        return tensor

    def wait_for_everyone(self) -> None:
        if self.num_processes > 1:
            dist.barrier()

    def unwrap_model(self, model):
        return model

    def print(self, *a, **k):
        if self.is_main_process:
            print(*a, **k)
