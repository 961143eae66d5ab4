"""Online-data-mixing plugin - configuration path ``training.odm.odm`` (``update_interval``, ``sampling_interval``,
``reward_type``, ``gamma``, ``eta``, ``resume_from_checkpoint``); lifecycle of
fms_acceleration_odm/framework_plugin_odm.py:30-86: the augmentation stashes the user's ``eval_steps`` on the model
and forces evaluation hooks to fire every step, the callback stage installs the trainer hooks and the loader-state
saving callback."""
from __future__ import annotations

from typing import Dict, Tuple

import torch

from ...framework.framework_plugin import AccelerationPlugin
from .callback import DataloaderSavingCallback
from .patch import patch_hf_trainer_evaluate


class OnlineDataMixingAccelerationPlugin(AccelerationPlugin):
    def __init__(self, configurations: Dict[str, Dict]):
        super().__init__(configurations)
        self._update_interval = self._check_config_and_maybe_check_values(key="training.odm.odm.update_interval", default=1)
        self._resume_from_checkpoint = self._check_config_and_maybe_check_values(
            key="training.odm.odm.resume_from_checkpoint", default=False)

    @property
    def requires_augmentation(self):
        return True

    def augmentation(self, model, train_args, modifiable_args: Tuple):
        model.ta_eval_steps = train_args.eval_steps
        train_args.eval_steps = 1
        train_args.eval_strategy = "steps"
        model.ta_update_interval = self._update_interval
        model.resume_from_checkpoint = self._resume_from_checkpoint
        return model, modifiable_args

    def get_callbacks_and_ready_for_train(self, model: torch.nn.Module = None, accelerator=None):
        patch_hf_trainer_evaluate()
        return [DataloaderSavingCallback(accelerator)]


AccelerationPlugin.register_plugin(OnlineDataMixingAccelerationPlugin, configuration_and_paths=["training.odm.odm"])
