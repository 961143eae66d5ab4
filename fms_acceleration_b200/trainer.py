"""Training harness: synthetic packed batches, AdamW step, device-side timing.

The reference has no training loop of its own (it plugs into HF Trainer); this harness is what drives the
plugin lifecycle here: ``AccelerationFramework.model_loader -> augmentation ->
get_callbacks_and_ready_for_train`` followed by ``Trainer.train_step`` per batch.
"""
from __future__ import annotations

import math
import os
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional

import torch
from torch import nn


@dataclass
class TrainArgs:
    """The subset of HF ``TrainingArguments`` that plugins read."""

    per_device_train_batch_size: int = 4
    gradient_accumulation_steps: int = 1
    learning_rate: float = 1e-4
    weight_decay: float = 0.0
    max_grad_norm: float = 0.0
    bf16: bool = False
    fp16: bool = False
    gradient_checkpointing: bool = False
    gradient_checkpointing_kwargs: Optional[dict] = None
    seed: int = 0
    max_seq_length: int = 4096
    output_dir: str = "./out"
    eval_steps: Optional[int] = None
    eval_strategy: str = "no"
    logging_steps: int = 1
    save_steps: int = 0
    padding_free: bool = True
    world_size: int = 1
    parallel_mode: str = "NOT_DISTRIBUTED"


def synthetic_packed_batch(vocab_size: int, batch_size: int, seq_len: int, doc_len_range=(128, 4096), seed: int = 0,
                           pin: bool = True) -> Dict[str, torch.Tensor]:
    """One padding-free batch of ``batch_size * seq_len`` uniform-random tokens made of documents whose lengths
    are uniform in ``doc_len_range`` (the last document of each row is cut at the row end).  Host tensors
    (pinned when requested): ``input_ids``, ``position_ids``, ``labels`` of shape [1, T] and ``cu_seqlens``."""
    g = torch.Generator().manual_seed(seed)
    T = batch_size * seq_len
    lo, hi = doc_len_range
    lens: List[int] = []
    for _ in range(batch_size):
        left = seq_len
        while left > 0:
            n = int(torch.randint(lo, hi + 1, (1,), generator=g).item())
            n = min(n, left)
            lens.append(n)
            left -= n
    cu = torch.zeros(len(lens) + 1, dtype=torch.int32)
    cu[1:] = torch.tensor(lens, dtype=torch.int32).cumsum(0)
    ids = torch.randint(0, vocab_size, (1, T), generator=g, dtype=torch.int64)
    pos = torch.cat([torch.arange(n, dtype=torch.int64) for n in lens])[None]
    labels = ids.clone()
    labels[0, cu[:-1].long()] = -100  # the first token of every document is never a target
    out = {"input_ids": ids, "position_ids": pos, "labels": labels, "cu_seqlens": cu}
    if pin and torch.cuda.is_available():
        out = {k: v.pin_memory() for k, v in out.items()}
    return out


def to_device(batch: Dict[str, torch.Tensor], device) -> Dict[str, torch.Tensor]:
    return {k: v.to(device, non_blocking=True) for k, v in batch.items()}


class Trainer:
    """Minimal single-process-per-GPU trainer.

    ``engine`` (optional) is the sharded-parameter / gradient-synchronisation engine from
    :mod:`fms_acceleration_b200.parallel`; without it the trainer is plain single-GPU (or CPU).
    """

    def __init__(self, model: nn.Module, args: TrainArgs, optimizer: Optional[torch.optim.Optimizer] = None,
                 engine=None, callbacks: Optional[list] = None):
        self.model = model
        self.args = args
        self.engine = engine
        self.callbacks = callbacks or []
        params = [p for p in model.parameters() if p.requires_grad]
        if optimizer is None:
            fused = bool(params) and params[0].is_cuda
            optimizer = torch.optim.AdamW(params, lr=args.learning_rate, weight_decay=args.weight_decay, fused=fused)
        self.optimizer = optimizer
        self.params = params
        self.global_step = 0
        self.log_history: List[dict] = []

    def device(self):
        for p in self.model.parameters():
            return p.device
        for b in self.model.buffers():
            return b.device
        return torch.device("cpu")

    def train_step(self, batch: Dict[str, torch.Tensor]) -> torch.Tensor:
        """One optimizer step on one (host or device) batch; returns the detached loss (device tensor)."""
        dev = self.device()
        if batch["input_ids"].device != dev:
            batch = to_device(batch, dev)
        self.model.train()
        kwargs = dict(input_ids=batch["input_ids"], labels=batch["labels"])
        if "position_ids" in batch:
            kwargs["position_ids"] = batch["position_ids"]
        if "cu_seqlens" in batch and getattr(self.args, "padding_free", False):
            kwargs["cu_seqlens"] = batch["cu_seqlens"]
            kwargs.pop("position_ids", None)
        out = self.model(**kwargs)
        loss = out.loss
        loss.backward()
        if self.engine is not None:
            self.engine.reduce_gradients()
        if self.args.max_grad_norm and self.args.max_grad_norm > 0:
            torch.nn.utils.clip_grad_norm_(self.params, self.args.max_grad_norm)
        self.optimizer.step()
        if self.engine is not None:
            self.engine.zero_grad()
        else:
            self.optimizer.zero_grad(set_to_none=True)
        self.global_step += 1
        return loss.detach()

    def train(self, batches, max_steps: Optional[int] = None):
        losses = []
        for i, b in enumerate(batches):
            if max_steps is not None and i >= max_steps:
                break
            loss = self.train_step(b)
            losses.append(float(loss))
            self.log_history.append({"step": self.global_step, "loss": losses[-1]})
        return losses
