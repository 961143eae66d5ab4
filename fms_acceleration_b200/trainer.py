"""Training harness: synthetic packed batches, AdamW step, device-side timing.

The reference has no training loop of its own (it plugs into HF Trainer); this harness is what drives the
plugin lifecycle here: ``AccelerationFramework.model_loader -> augmentation ->
get_callbacks_and_ready_for_train`` followed by ``Trainer.train_step`` per batch.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Dict, List, Optional

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


def _adamw(params, lr: float, weight_decay: float) -> torch.optim.Optimizer:
    """AdamW for ``params``: the in-tree kernel on a GPU (``FMSB_ADAMW=torch`` keeps torch's fused one), torch's on a CPU."""
    on_gpu = bool(params) and params[0].is_cuda
    if on_gpu and os.environ.get("FMSB_ADAMW", "native") != "torch":
        from .ops.optim import AdamW

        return AdamW(params, lr=lr, weight_decay=weight_decay)
    return torch.optim.AdamW(params, lr=lr, weight_decay=weight_decay, fused=on_gpu)


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
        if optimizer is None and engine is not None and getattr(engine, "shard_optimizer", False) \
                and hasattr(engine, "flat_params"):
            # optimizer states of the replicated parameters sharded over the ranks (the engine owns the flat parameter
            # and gradient buffers); expert-parallel parameters, already disjoint over the ranks, get a plain AdamW
            optimizer = engine.build_optimizer(args.learning_rate, args.weight_decay)
            if engine.ep_params:
                optimizer.ep_optimizer = _adamw(engine.ep_params, args.learning_rate, args.weight_decay)
        if optimizer is None:
            optimizer = _adamw(params, args.learning_rate, args.weight_decay)
        self.optimizer = optimizer
        self.params = params
        self.global_step = 0
        self.log_history: List[dict] = []
        self._micro = 0          # micro-batches accumulated since the last optimizer step
        self._status = None      # asynchronous view of the device status word (GPU runs only)
        if getattr(args, "gradient_checkpointing", False):
            base = model.get_base_model() if hasattr(model, "get_base_model") else model
            if hasattr(base, "gradient_checkpointing_enable"):
                base.gradient_checkpointing_enable(getattr(args, "gradient_checkpointing_kwargs", None))

    def device(self):
        for p in self.model.parameters():
            return p.device
        for b in self.model.buffers():
            return b.device
        return torch.device("cpu")

    def _has_expert_parallel(self) -> bool:
        return any(getattr(p, "_fmsb_expert_parallel", False) for p in self.params)

    def train_step(self, batch: Dict[str, torch.Tensor]) -> torch.Tensor:
        """Forward + backward of one (host or device) batch; every ``gradient_accumulation_steps``-th call also
        reduces the gradients across ranks, clips, and steps the optimizer.  Returns the detached loss (device
        tensor) of this batch."""
        dev = self.device()
        if dev.type == "cuda":
            if self._status is None:
                from . import _native as NV

                self._status = NV.StatusMonitor(dev)
            # a kernel of an EARLIER step whose bounded wait ran out left its code in the status word; raise it here
            # (no host synchronisation: the snapshot is only looked at once its copy has completed)
            self._status.raise_if_set()
        if batch["input_ids"].device != dev:
            batch = to_device(batch, dev)
        self.model.train()
        kwargs = dict(input_ids=batch["input_ids"], labels=batch["labels"])
        if "position_ids" in batch:
            kwargs["position_ids"] = batch["position_ids"]
        if "cu_seqlens" in batch and getattr(self.args, "padding_free", False):
            kwargs["cu_seqlens"] = batch["cu_seqlens"]
            kwargs.pop("position_ids", None)
        accum = max(1, int(getattr(self.args, "gradient_accumulation_steps", 1) or 1))
        last = (self._micro + 1) % accum == 0
        if self.engine is not None:
            self.engine.begin_micro_step(last)
        out = self.model(**kwargs)
        loss = out.loss
        (loss / accum if accum > 1 else loss).backward()
        if self.engine is not None:
            self.engine.end_micro_step()
        self._micro += 1
        if not last:
            return loss.detach()
        self._micro = 0
        sharded = self.engine is not None and self.optimizer is getattr(self.engine, "sharded_optimizer", None) \
            and self.optimizer is not None
        if self.engine is not None:
            self.engine.reduce_gradients()
        if sharded:
            self.optimizer.max_grad_norm = self.args.max_grad_norm or 0.0  # clipped on the reduced slices
        elif self.args.max_grad_norm and self.args.max_grad_norm > 0:
            if self._has_expert_parallel():
                # expert shards differ per rank: their squared norms are summed over the expert-parallel group, so
                # that every rank scales by the same factor
                from .plugins.moe.utils.checkpoint_utils import clip_grad_norm_

                clip_grad_norm_(self.params, self.args.max_grad_norm)
            else:
                torch.nn.utils.clip_grad_norm_(self.params, self.args.max_grad_norm)
        self.optimizer.step()
        if self.engine is not None:
            self.engine.zero_grad()
            if sharded and self.optimizer.ep_optimizer is not None:
                self.optimizer.ep_optimizer.zero_grad(set_to_none=True)
        else:
            self.optimizer.zero_grad(set_to_none=True)
        self.global_step += 1
        if self._status is not None:
            self._status.poll()
        return loss.detach()

    def train(self, batches, max_steps: Optional[int] = None):
        losses = []
        for i, b in enumerate(batches):
            if max_steps is not None and i >= max_steps:
                break
            loss = self.train_step(b)
            losses.append(float(loss))
            self.log_history.append({"step": self.global_step, "loss": losses[-1]})
            if self.args.save_steps and self.global_step % self.args.save_steps == 0:
                self.save_checkpoint()
        return losses

    # ------------------------------------------------------------------ checkpoint / resume
    def _is_lora(self) -> bool:
        return any("lora_" in n for n, _ in self.model.named_parameters())

    def save_checkpoint(self, output_dir: Optional[str] = None, scheduler=None) -> str:
        """Write ``<output_dir>/checkpoint-<step>/``: the model (only the adapters for a LoRA run) and the optimizer as
        torch distributed-checkpoint directories named like accelerate's FSDP checkpoints
        (``pytorch_model_fsdp_0`` / ``optimizer_0``, cf. fms_acceleration_moe/utils/checkpoint_utils.py:129-158 of the
        reference), ``trainer_state.json``, per-rank RNG state, and for LoRA runs a PEFT-style
        ``adapter_model.safetensors`` + ``adapter_config.json``.  Callbacks get ``on_save`` (the data-mixing plugin
        stores its loader state there)."""
        import json

        from .plugins.moe.utils import checkpoint_utils as CU

        rank = torch.distributed.get_rank() if torch.distributed.is_available() and torch.distributed.is_initialized() else 0
        root = output_dir or self.args.output_dir
        ckpt = os.path.join(root, f"checkpoint-{self.global_step}")
        os.makedirs(ckpt, exist_ok=True)
        lora = self._is_lora()
        CU.save_fsdp_model(None, None, self.model, ckpt, 0)
        # a rank-sharded optimizer hands its slices over as shards of group-wide tensors, expert-parallel parameters
        # and their moments likewise: one checkpoint directory holds the whole state whatever the layout
        CU.save_fsdp_optimizer(None, None, self.optimizer, self.model, ckpt, 0, lora_only=lora)
        torch.save({"cpu": torch.get_rng_state(),
                    "cuda": torch.cuda.get_rng_state() if torch.cuda.is_available() else None},
                   os.path.join(ckpt, f"rng_state_{rank}.pth"))
        if rank == 0:
            with open(os.path.join(ckpt, "trainer_state.json"), "w", encoding="utf-8") as fh:
                json.dump({"global_step": self.global_step, "log_history": self.log_history}, fh, indent=1)
            if scheduler is not None:
                torch.save(scheduler.state_dict(), os.path.join(ckpt, "scheduler.pt"))
            if lora:
                from safetensors.torch import save_file

                # PEFT's file layout: adapter tensors without the adapter name in their keys
                src = (self.model.adapter_state_dict() if hasattr(self.model, "adapter_state_dict") else
                       {k.replace(".default", ""): v for k, v in self.model.state_dict().items() if "lora_" in k})
                sd = {k: v.detach().cpu().contiguous() for k, v in src.items()}
                save_file(sd, os.path.join(ckpt, "adapter_model.safetensors"), metadata={"format": "pt"})
                cfg = getattr(self.model, "peft_config", None)
                cfg = cfg.get("default") if isinstance(cfg, dict) else cfg
                if cfg is not None and hasattr(cfg, "to_dict"):
                    with open(os.path.join(ckpt, "adapter_config.json"), "w", encoding="utf-8") as fh:
                        json.dump(cfg.to_dict(), fh, indent=1)
        state = type("State", (), {"global_step": self.global_step})()
        for cb in self.callbacks:
            if hasattr(cb, "on_save"):
                cb.on_save(self.args, state, None)
        return ckpt

    def load_checkpoint(self, ckpt: str, scheduler=None) -> None:
        """Resume model (or adapters), optimizer, step counter, log history and RNG state from ``save_checkpoint``."""
        import json

        from .plugins.moe.utils import checkpoint_utils as CU

        rank = torch.distributed.get_rank() if torch.distributed.is_available() and torch.distributed.is_initialized() else 0
        from torch.distributed.checkpoint.api import CheckpointException

        try:
            CU.load_fsdp_model(None, None, self.model, ckpt, 0)
            CU.load_fsdp_optimizer(None, None, self.optimizer, self.model, ckpt, 0, lora_only=self._is_lora())
        except CheckpointException as exc:  # derives from BaseException: turn it into an ordinary error
            raise RuntimeError(f"checkpoint {ckpt!r} is incomplete or damaged: {str(exc).splitlines()[0]}") from exc
        with open(os.path.join(ckpt, "trainer_state.json"), encoding="utf-8") as fh:
            st = json.load(fh)
        self.global_step = int(st["global_step"])
        self.log_history = list(st.get("log_history", []))
        rng_file = os.path.join(ckpt, f"rng_state_{rank}.pth")
        if os.path.exists(rng_file):
            rng = torch.load(rng_file, weights_only=False)
            torch.set_rng_state(rng["cpu"])
            if rng.get("cuda") is not None and torch.cuda.is_available():
                torch.cuda.set_rng_state(rng["cuda"])
        if scheduler is not None and os.path.exists(os.path.join(ckpt, "scheduler.pt")):
            scheduler.load_state_dict(torch.load(os.path.join(ckpt, "scheduler.pt"), weights_only=False))

    @staticmethod
    def latest_checkpoint(output_dir: str) -> Optional[str]:
        best, best_step = None, -1
        if os.path.isdir(output_dir):
            for name in os.listdir(output_dir):
                if name.startswith("checkpoint-") and name[11:].isdigit() and int(name[11:]) > best_step:
                    best, best_step = os.path.join(output_dir, name), int(name[11:])
        return best
