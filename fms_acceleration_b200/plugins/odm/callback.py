"""Checkpoint hook: store the mixing data loader's state as ``odm_dl_state_dict.bin`` inside
``checkpoint-<step>/`` (behaviour of fms_acceleration_odm/callback.py:14-38).  Duck-typed: works as a Hugging Face
``TrainerCallback`` and with this package's trainer (both call ``on_save(args, state, control)``)."""
from __future__ import annotations

import os

import torch

STATE_FILE = "odm_dl_state_dict.bin"

try:  # be a real TrainerCallback when transformers is importable
    from transformers import TrainerCallback as _Base
except Exception:  # pragma: no cover
    _Base = object


class DataloaderSavingCallback(_Base):
    def __init__(self, accelerator):
        super().__init__()
        self.accelerator = accelerator

    def _stateful_loaders(self):
        for dl in getattr(self.accelerator, "_dataloaders", []) or []:
            target = getattr(dl, "base_dataloader", dl)
            ds = getattr(target, "dataset", None)
            if hasattr(dl, "state_dict") or hasattr(ds, "state_dict"):
                yield dl, ds

    def on_save(self, args, state, control=None, **kwargs):
        if not getattr(self.accelerator, "is_main_process", True):
            return
        ckpt = os.path.join(args.output_dir, f"checkpoint-{state.global_step}")
        os.makedirs(ckpt, exist_ok=True)
        for dl, ds in self._stateful_loaders():
            sd = dl.state_dict() if hasattr(dl, "state_dict") else {"dataset_state": ds.state_dict()}
            torch.save(sd, os.path.join(ckpt, STATE_FILE))
            break
