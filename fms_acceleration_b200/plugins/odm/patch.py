"""Hooks that make a Hugging Face ``Trainer`` drive the bandit (role of fms_acceleration_odm/patch.py:9-233):

* ``_evaluate`` runs the user's evaluation only every ``model.ta_eval_steps`` steps and a bandit update every
  ``model.ta_update_interval`` steps (the plugin forces ``eval_steps = 1`` so that the hook fires every step);
* ``get_train_dataloader`` restores ``odm_dl_state_dict.bin`` when resuming; ``skip_first_batches`` becomes a no-op
  because the restored loader already points at the right sample.

All patches are applied only when ``transformers`` is importable; this package's own trainer calls
``maybe_update_sampling_weights`` directly.
"""
from __future__ import annotations

import os

import torch

from .callback import STATE_FILE


def maybe_update_sampling_weights(model, train_dataset, accelerator, state) -> bool:
    """Bandit update when the step count says so; returns whether an update ran."""
    interval = getattr(model, "ta_update_interval", None)
    if not interval or state.global_step % interval != 0 or not hasattr(train_dataset, "update_sampling_weights"):
        return False
    was_training = model.training
    model.eval()
    try:
        train_dataset.update_sampling_weights(model, accelerator, state)
    finally:
        model.train(was_training)
    return True


def _evaluate(self, trial, ignore_keys_for_eval, skip_scheduler=False):
    metrics = None
    if self.model.ta_eval_steps and self.state.global_step % self.model.ta_eval_steps == 0:
        metrics = self.evaluate(ignore_keys=ignore_keys_for_eval)
        self._report_to_hp_search(trial, self.state.global_step, metrics)
        plateau = torch.optim.lr_scheduler.ReduceLROnPlateau
        if isinstance(self.lr_scheduler, plateau) and not skip_scheduler:
            name = self.args.metric_for_best_model
            name = name if name.startswith("eval_") else f"eval_{name}"
            if name not in metrics:
                raise KeyError(f"The `metric_for_best_model` training argument is set to '{name}', which is not found in "
                               f"the evaluation metrics. The available evaluation metrics are: {list(metrics.keys())}.")
            self.lr_scheduler.step(metrics[name])
    maybe_update_sampling_weights(self.model, self.train_dataset, self.accelerator, self.state)
    return metrics


def restore_dataloader_state(dataloader, resume_dir: str) -> bool:
    path = os.path.join(resume_dir, STATE_FILE)
    if not os.path.exists(path):
        return False
    sd = torch.load(path, weights_only=False)
    if hasattr(dataloader, "load_state_dict"):
        dataloader.load_state_dict(sd)
    elif "dataset_state" in sd and hasattr(dataloader.dataset, "load_state_dict"):
        dataloader.dataset.load_state_dict(sd["dataset_state"])
    return True


def skip_first_batches(dataloader, num_batches=0):
    """Replacement for ``transformers.trainer.skip_first_batches``: the restored loader already points at the next
    sample, so nothing is skipped (fms_acceleration_odm/patch.py:232-233)."""
    return dataloader


def get_train_dataloader(self):
    """Replacement for ``Trainer.get_train_dataloader`` (fms_acceleration_odm/patch.py:187-229): build the loader the
    stock way, then, when ``model.resume_from_checkpoint`` names a checkpoint (``True`` = the last one under
    ``args.output_dir``), restore the loader / dataset state saved there."""
    if self.train_dataset is None:
        raise ValueError("Trainer: training requires a train_dataset.")
    original = getattr(type(self), "_fmsb_original_get_train_dataloader", None)
    if original is not None:
        dl = original(self)
    else:
        dl = self._get_dataloader(dataset=self.train_dataset, description="Training", batch_size=self._train_batch_size,
                                  sampler_fn=self._get_train_sampler, is_training=True)
    resume = getattr(self.model, "resume_from_checkpoint", None)
    if resume is True:
        from transformers.trainer_utils import get_last_checkpoint

        resume = get_last_checkpoint(self.args.output_dir)
        if resume is None:
            raise ValueError(f"No valid checkpoint found in output directory ({self.args.output_dir})")
        self.model.resume_from_checkpoint = resume
    if isinstance(resume, str) and os.path.isdir(resume):
        restore_dataloader_state(dl, resume)
    return dl


def patch_hf_trainer_evaluate() -> bool:
    """Install the hooks on ``transformers.Trainer``.  Returns False when transformers is not available."""
    try:
        from transformers import Trainer
    except Exception:
        return False
    from ...framework.model_patcher import patch_target_module

    patch_target_module("transformers.trainer.Trainer._evaluate", _evaluate)
    if not hasattr(Trainer, "_fmsb_original_get_train_dataloader"):
        Trainer._fmsb_original_get_train_dataloader = Trainer.get_train_dataloader
    Trainer.get_train_dataloader = get_train_dataloader
    try:
        import transformers.trainer as tr

        tr.skip_first_batches = skip_first_batches
    except Exception:
        pass
    return True
