"""One fine-tuning run from command-line arguments: the program every benchmark experiment launches.

The reference benchmarks drive an external trainer (``python -m tuning.sft_trainer`` from fms-hf-tuning,
scripts/benchmarks/benchmark.py:34) with HF ``TrainingArguments`` names.  This module is the in-tree counterpart:
the same argument names where they exist, the acceleration framework configured from
``--acceleration_framework_config_file`` or ``ACCELERATION_FRAMEWORK_CONFIG_FILE``, and the same kind of stdout
(a dict per logging step and one final dict with ``train_runtime`` / ``train_tokens_per_second`` / ``train_loss``)
so that the harness can scrape it.

    python -m fms_acceleration_b200.benchmarks.sft_trainer --model_name_or_path mistral-7b --peft_method lora \
        --r 16 --lora_alpha 16 --target_modules q_proj k_proj v_proj o_proj --max_steps 100 \
        --per_device_train_batch_size 4 --max_seq_length 4096 \
        --acceleration_framework_config_file sample-configurations/accelerated-peft-bnb-nf4-foak-...yaml

Several GPUs: launch with ``python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 -m
fms_acceleration_b200.benchmarks.sft_trainer ...``.  Without ``--training_data_path`` the data are synthetic packed
documents; with it, a JSON/JSONL file of ``{"input_ids": [...], "labels": [...]}`` rows is read.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys
import time
from typing import Dict, List, Optional

import torch

from ..framework.constants import ACCELERATION_FRAMEWORK_ENV_KEY as ENV_CONFIG_FILE


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    tf = lambda s: str(s).lower() in ("1", "true", "yes")  # noqa: E731
    ap.add_argument("--model_name_or_path", required=True)
    ap.add_argument("--acceleration_framework_config_file", default=None)
    ap.add_argument("--torch_dtype", default="bfloat16", choices=["bfloat16", "float16", "float32"])
    ap.add_argument("--bf16", type=tf, nargs="?", const=True, default=False)
    ap.add_argument("--fp16", type=tf, nargs="?", const=True, default=False)
    ap.add_argument("--peft_method", default="none", choices=["none", "lora"])
    # ``--lora_r`` is the spelling the benchmark runner uses under torch.distributed.run, whose own parser rejects a
    # bare ``--r`` in the trainer's arguments as an ambiguous abbreviation of its ``--rdzv-*`` / ``--role`` options
    ap.add_argument("--r", "--lora_r", dest="r", type=int, default=16)
    ap.add_argument("--lora_alpha", type=int, default=16)
    ap.add_argument("--lora_dropout", type=float, default=0.0)
    ap.add_argument("--target_modules", nargs="*", default=["q_proj", "k_proj", "v_proj", "o_proj"])
    ap.add_argument("--per_device_train_batch_size", type=int, default=4)
    ap.add_argument("--gradient_accumulation_steps", type=int, default=1)
    ap.add_argument("--max_seq_length", type=int, default=4096)
    ap.add_argument("--max_steps", type=int, default=100)
    ap.add_argument("--num_train_epochs", type=float, default=1.0)
    ap.add_argument("--learning_rate", type=float, default=2e-4)
    ap.add_argument("--weight_decay", type=float, default=0.01)
    ap.add_argument("--adam_epsilon", type=float, default=1e-8)
    ap.add_argument("--warmup_steps", type=int, default=10)
    ap.add_argument("--lr_scheduler_type", default="linear", choices=["linear", "constant", "cosine"])
    ap.add_argument("--max_grad_norm", type=float, default=1.0)
    ap.add_argument("--logging_steps", type=int, default=10)
    ap.add_argument("--logging_strategy", default="steps")
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--training_data_path", default=None)
    ap.add_argument("--packing", type=tf, nargs="?", const=True, default=False)
    ap.add_argument("--padding_free", nargs="*", default=None)
    ap.add_argument("--output_dir", default="./out")
    ap.add_argument("--skip_memory_metrics", type=tf, nargs="?", const=True, default=True)
    ap.add_argument("--include_tokens_per_second", type=tf, nargs="?", const=True, default=True)
    ap.add_argument("--save_strategy", default="no", choices=["no", "steps", "epoch"],
                    help="steps: a checkpoint every --save_steps steps; epoch: one at the end of the run")
    ap.add_argument("--save_steps", type=int, default=500)
    ap.add_argument("--resume_from_checkpoint", default=None,
                    help="a checkpoint directory, or True for the newest one under --output_dir")
    ap.add_argument("--gradient_checkpointing", type=tf, nargs="?", const=True, default=False,
                    help="recompute every decoder layer in backward (the reference's benchmark default)")
    # arguments of the reference's benchmark defaults that have nothing to switch here: attention is always the
    # in-tree variable-length kernel, there is no evaluation loop, and the training file is already tokenised and
    # masked by data_processing.py (which is where the response template and the text field are used)
    ap.add_argument("--use_flash_attn", type=tf, nargs="?", const=True, default=True)
    ap.add_argument("--evaluation_strategy", "--eval_strategy", dest="evaluation_strategy", default="no")
    ap.add_argument("--response_template", default=None)
    ap.add_argument("--dataset_text_field", default=None)
    ap.add_argument("--num_layers_override", type=int, default=0, help="debugging: shrink the model")
    return ap


def lr_lambda(kind: str, warmup: int, total: int):
    def f(step: int) -> float:
        if step < warmup:
            return (step + 1) / max(1, warmup)
        if kind == "constant":
            return 1.0
        frac = (step - warmup) / max(1, total - warmup)
        if kind == "cosine":
            return 0.5 * (1.0 + math.cos(math.pi * min(1.0, frac)))
        return max(0.0, 1.0 - frac)

    return f


def load_token_rows(path: str) -> List[Dict[str, List[int]]]:
    rows = []
    with open(path, encoding="utf-8") as fh:
        head = fh.read(1)
        fh.seek(0)
        if head == "[":
            rows = json.load(fh)
        else:
            rows = [json.loads(line) for line in fh if line.strip()]
    for r in rows:
        if "labels" not in r:
            r["labels"] = list(r["input_ids"])
    return rows


class PackedRows:
    """Greedy padding-free batches of at most ``batch * seq_len`` tokens from tokenised rows."""

    def __init__(self, rows, batch: int, seq_len: int, seed: int, rank: int, world: int):
        from ..plugins.aadp.aadp_utils import DataCollatorWithFlattening

        # longer samples are cut at the maximum sequence length (what the reference's trainer does with them)
        self.rows = [r if len(r["input_ids"]) <= seq_len else
                     {"input_ids": r["input_ids"][:seq_len], "labels": r["labels"][:seq_len]} for r in rows]
        if not self.rows:
            raise ValueError("the training file holds no samples")
        self.cap = batch * seq_len
        self.collate = DataCollatorWithFlattening(return_cu_seqlens=True)
        g = torch.Generator().manual_seed(seed)
        order = torch.randperm(len(self.rows), generator=g).tolist()
        self.order = order[rank::world]
        self.pos = 0

    def next(self):
        feats, n = [], 0
        while True:
            if self.pos >= len(self.order):
                self.pos = 0
            r = self.rows[self.order[self.pos]]
            if feats and n + len(r["input_ids"]) > self.cap:
                break
            feats.append({"input_ids": r["input_ids"], "labels": r["labels"]})
            n += len(r["input_ids"])
            self.pos += 1
        return self.collate(feats)  # tensors of shape [1, total tokens] plus cu_seqlens


def main(argv: Optional[List[str]] = None) -> int:
    args, unknown = build_parser().parse_known_args(argv)
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    cuda = torch.cuda.is_available()
    dev = torch.device("cuda", local_rank) if cuda else torch.device("cpu")
    if cuda:
        torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl" if cuda else "gloo", **({"device_id": dev} if cuda else {}))
    if unknown and rank == 0:
        print(f"ignored arguments: {unknown}", file=sys.stderr)

    import fms_acceleration_b200.plugins  # noqa: F401  (registers the plugins)
    from ..compat import Accelerator
    from ..framework import AccelerationFramework
    from ..models.builder import build_model, resolve_config
    from ..nn import LoraConfig, get_peft_model
    from ..trainer import TrainArgs, Trainer, synthetic_packed_batch

    dtype = {"bfloat16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32}[args.torch_dtype]
    if not cuda:
        dtype = torch.float32
    cfg = resolve_config(args.model_name_or_path)
    if args.num_layers_override:
        cfg.num_hidden_layers = args.num_layers_override
    cfg_file = args.acceleration_framework_config_file or os.environ.get(ENV_CONFIG_FILE)
    framework = AccelerationFramework(cfg_file) if cfg_file else None
    targs = TrainArgs(per_device_train_batch_size=args.per_device_train_batch_size,
                      gradient_accumulation_steps=args.gradient_accumulation_steps, learning_rate=args.learning_rate,
                      weight_decay=args.weight_decay, max_grad_norm=args.max_grad_norm,
                      # mixed precision as asked for on the command line, or implied by the model dtype
                      bf16=bool(args.bf16) or dtype == torch.bfloat16,
                      fp16=(bool(args.fp16) or dtype == torch.float16) and not bool(args.bf16),
                      seed=args.seed, max_seq_length=args.max_seq_length, output_dir=args.output_dir,
                      logging_steps=args.logging_steps, padding_free=True, world_size=world,
                      gradient_checkpointing=bool(args.gradient_checkpointing),
                      parallel_mode="DISTRIBUTED" if world > 1 else "NOT_DISTRIBUTED")
    torch.manual_seed(args.seed)
    if cuda:
        torch.cuda.reset_peak_memory_stats()
    t_load = time.perf_counter()
    # a checkpoint directory is handed over as such (the loaders read its weights); a preset as its configuration
    source = args.model_name_or_path if os.path.isdir(str(args.model_name_or_path)) and not args.num_layers_override else cfg
    if framework is not None and framework.requires_custom_loading:
        model = framework.model_loader(source, torch_dtype=dtype, device=dev)
    else:
        model = build_model(source, device=dev, dtype=dtype, seed=args.seed)
    peft_config = None
    if args.peft_method == "lora":
        peft_config = LoraConfig(r=args.r, lora_alpha=args.lora_alpha, lora_dropout=args.lora_dropout,
                                 target_modules=list(args.target_modules))
    if framework is not None and framework.requires_augmentation:
        model, (peft_config,) = framework.augmentation(model, targs, modifiable_args=(peft_config,))
    if peft_config is not None:
        model = get_peft_model(model, peft_config)
    accelerator = Accelerator(device=dev)
    callbacks = framework.get_callbacks_and_ready_for_train(model, accelerator) if framework is not None else []
    engine = getattr(accelerator, "engine", None)
    if engine is None and world > 1:
        from ..parallel.engine import install_engine

        engine = install_engine(model, accelerator)
    load_s = time.perf_counter() - t_load

    params = [p for p in model.parameters() if p.requires_grad]
    opt = torch.optim.AdamW(params, lr=args.learning_rate, weight_decay=args.weight_decay, eps=args.adam_epsilon,
                            fused=bool(params) and params[0].is_cuda)
    sched = torch.optim.lr_scheduler.LambdaLR(opt, lr_lambda(args.lr_scheduler_type, args.warmup_steps, args.max_steps))
    trainer = Trainer(model, targs, optimizer=opt, engine=engine, callbacks=callbacks)

    if args.training_data_path:
        rows = load_token_rows(args.training_data_path)
        source = PackedRows(rows, args.per_device_train_batch_size, args.max_seq_length, args.seed, rank, world)
        next_batch = source.next
    else:
        counter = [0]

        def next_batch():
            counter[0] += 1
            return synthetic_packed_batch(cfg.vocab_size, args.per_device_train_batch_size, args.max_seq_length,
                                          (min(128, args.max_seq_length), args.max_seq_length),
                                          seed=1000 * rank + counter[0], pin=cuda)

    def sync():
        if world > 1:
            dist.barrier()
        if cuda:
            torch.cuda.synchronize()

    first_step = 1
    accum = max(1, int(args.gradient_accumulation_steps or 1))
    if args.resume_from_checkpoint:
        ckpt = args.resume_from_checkpoint
        if str(ckpt).lower() == "true":
            ckpt = Trainer.latest_checkpoint(args.output_dir)
            if ckpt is None:
                raise ValueError(f"No valid checkpoint found in output directory ({args.output_dir})")
        trainer.load_checkpoint(ckpt, scheduler=sched)
        first_step = trainer.global_step * accum + 1  # the loop counts micro-batches, the trainer optimizer steps
        for _ in range(first_step - 1):  # the data stream continues where the saved run stopped
            next_batch()

    sync()
    t0 = time.perf_counter()
    tokens = 0
    run_loss, n_log = 0.0, 0
    total_loss = 0.0
    for step in range(first_step, args.max_steps + 1):
        batch = next_batch()
        tokens += int(batch["input_ids"].numel())
        loss = trainer.train_step(batch)
        sched.step()
        boundary = step % accum == 0  # checkpoints are taken between optimizer steps only
        if boundary and ((args.save_strategy == "steps" and (step // accum) % args.save_steps == 0) or
                         (args.save_strategy == "epoch" and step + accum > args.max_steps)):
            trainer.save_checkpoint(args.output_dir, scheduler=sched)
        run_loss += float(loss)
        n_log += 1
        if args.logging_strategy == "steps" and step % args.logging_steps == 0 and rank == 0:
            print({"loss": round(run_loss / n_log, 4), "learning_rate": sched.get_last_lr()[0],
                   "epoch": round(step / args.max_steps, 2)}, flush=True)
            total_loss += run_loss
            run_loss, n_log = 0.0, 0
    total_loss += run_loss
    sync()
    runtime = time.perf_counter() - t0
    stats = torch.tensor([runtime, float(tokens)], dtype=torch.float64, device=dev)
    if world > 1:
        tmax = stats.clone()
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        dist.all_reduce(stats, op=dist.ReduceOp.SUM)
        runtime, tokens = float(tmax[0]), float(stats[1])
    if rank == 0:
        final = {
            "train_runtime": round(runtime, 4),
            "train_samples_per_second": round(args.max_steps * args.per_device_train_batch_size * world / runtime, 3),
            "train_steps_per_second": round(args.max_steps / runtime, 3),
            "train_tokens_per_second": round(tokens / runtime / world, 3),  # per device, as HF reports it
            "train_loss": round(total_loss / args.max_steps, 6),
            "epoch": 1.0,
            "model_load_time": round(load_s, 3),
        }
        if cuda and not args.skip_memory_metrics:
            final["train_mem_gpu_peaked_delta"] = 0
            final["mem_peak_torch_mem_alloc_in_bytes"] = int(torch.cuda.max_memory_allocated())
            final["mem_torch_mem_alloc_in_bytes"] = int(torch.cuda.memory_allocated())
        print(final, flush=True)
    if cuda:
        from .. import _native as NV

        NV.check_status()
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
