"""Mamba context-parallel plugin - configuration path ``training.mamba.cp`` (``degree``, ``mamba_impl`` default
``allgather``, ``mamba_recompute`` default False); lifecycle of fms_acceleration_mcp/framework_plugin_mcp.py:29-87."""
from __future__ import annotations

from typing import Dict, Tuple

import torch

from ...framework.framework_plugin import AccelerationPlugin
from .utils import patch_mamba_layers_with_cp_head


class MCPAccelerationPlugin(AccelerationPlugin):
    def __init__(self, configurations: Dict[str, Dict]):
        super().__init__(configurations)
        self._mamba_cp_degree = self._check_config_and_maybe_check_values(key="training.mamba.cp.degree", default=None)
        self._cp_mamba_impl = self._check_config_and_maybe_check_values(key="training.mamba.cp.mamba_impl",
                                                                        default="allgather")
        self._cp_mamba_recompute = self._check_config_and_maybe_check_values(key="training.mamba.cp.mamba_recompute",
                                                                             default=False)

    @property
    def requires_augmentation(self):
        return True

    def augmentation(self, model, train_args, modifiable_args: Tuple):
        if self._mamba_cp_degree is not None:
            rank, world_size = 0, 1
            if torch.distributed.is_available() and torch.distributed.is_initialized():
                rank = torch.distributed.get_rank()
                world_size = torch.distributed.get_world_size()
            patch_mamba_layers_with_cp_head(
                model=model, checkpoint_name_or_path=getattr(model.config, "name_or_path", None), rank=rank,
                cp_degree=self._mamba_cp_degree, world_size=world_size, cp_mamba_impl=self._cp_mamba_impl,
                cp_mamba_recompute=self._cp_mamba_recompute)
        return model, modifiable_args

    def get_callbacks_and_ready_for_train(self, model: torch.nn.Module = None, accelerator=None):
        if accelerator is not None and model is not None and next(model.parameters()).is_cuda \
                and getattr(accelerator, "num_processes", 1) > 1:
            from ...parallel.engine import install_engine

            # all parameters are replicated over the context-parallel ranks; gradients are SUMMED over them
            # (each rank holds the loss terms of its own slice, already divided by the global token count)
            install_engine(model, accelerator, shard_frozen=False, grad_scale=1.0)
        return []


AccelerationPlugin.register_plugin(MCPAccelerationPlugin, configuration_and_paths=["training.mamba.cp"])
