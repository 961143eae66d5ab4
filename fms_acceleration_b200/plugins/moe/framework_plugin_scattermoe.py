"""ScatterMoE plugin - configuration path ``training.moe.scattermoe`` (``ep_degree`` default 1,
``disable_distributed`` default False).

Same lifecycle as fms_acceleration_moe/framework_plugin_scattermoe.py:40-183 of the reference: the augmentation
swaps the sparse-MoE blocks for ScatterMoE modules (loading this rank's expert shard); at callback time the MoE
modules are excluded from parameter sharding and sharded checkpoints are forced.  Gradient synchronisation of
the experts (replicate dimension) and of all other parameters is done by this package's engine.
"""
from __future__ import annotations

from typing import Dict, Tuple

import torch

from ...framework.framework_plugin import AccelerationPlugin
from .utils import prepare_scattermoe
from .utils.scattermoe import ScatterMoE


class ScatterMoEAccelerationPlugin(AccelerationPlugin):
    restricted_model_archs = ["GraniteMoeForCausalLM", "MixtralForCausalLM", "GraniteMoeSharedForCausalLM",
                              "GraniteMoeHybridForCausalLM"]

    def __init__(self, configurations: Dict[str, Dict]):
        super().__init__(configurations)
        self._ep_degree = self._check_config_and_maybe_check_values(key="training.moe.scattermoe.ep_degree", default=1)
        self._disable_distributed = self._check_config_and_maybe_check_values(
            key="training.moe.scattermoe.disable_distributed", values=[True, False], default=False)

    @property
    def requires_augmentation(self):
        return True

    def augmentation(self, model, train_args, modifiable_args: Tuple):
        rank, world = 0, 1
        if torch.distributed.is_available() and torch.distributed.is_initialized():
            world = torch.distributed.get_world_size()
            rank = torch.distributed.get_rank()
        (peft_config,) = modifiable_args if len(modifiable_args) == 1 else (None,)
        budget = None
        bs, sl = getattr(train_args, "per_device_train_batch_size", None), getattr(train_args, "max_seq_length", None)
        if bs and sl:
            budget = int(bs) * int(sl)
        self._swapped = prepare_scattermoe(
            model, checkpoint_name_or_path=getattr(model.config, "name_or_path", None), rank=rank, world_size=world,
            ep_degree=self._ep_degree, disable_distributed=self._disable_distributed,
            mixed_precision=False, lora_config=peft_config, token_budget=budget)
        return model, modifiable_args

    def get_callbacks_and_ready_for_train(self, model: torch.nn.Module = None, accelerator=None):
        if accelerator is not None and getattr(accelerator.state, "fsdp_plugin", None) is not None and model is not None:
            plugin = accelerator.state.fsdp_plugin
            ignored = list(plugin.ignored_modules or [])
            ignored += [m for m in model.modules() if isinstance(m, ScatterMoE)]
            plugin.ignored_modules = ignored
            plugin.set_state_dict_type("SHARDED_STATE_DICT")
            if next(model.parameters()).is_cuda:
                from ...parallel.engine import install_engine

                install_engine(model, accelerator, shard_frozen=False)
        return []


AccelerationPlugin.register_plugin(ScatterMoEAccelerationPlugin, configuration_and_paths=["training.moe.scattermoe"])
