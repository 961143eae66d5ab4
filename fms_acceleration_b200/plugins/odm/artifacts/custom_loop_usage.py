"""Online data mixing in a hand-written training loop (no trainer class).

Counterpart of the reference's plugins/online-data-mixing/artifacts/custom_loop_usage.py:92-147: an
``OnlineMixingDataset`` over a few categories feeds a plain ``DataLoader``; every ``UPDATE_EVERY`` steps the bandit
weights are updated from a reward measured on the evaluation split of each category.

    python -m fms_acceleration_b200.plugins.odm.artifacts.custom_loop_usage [--steps 40] [--device cuda]

Runs on the CPU with the tiny Llama preset by default; all data are synthetic.
"""
from __future__ import annotations

import argparse
import tempfile

import torch
from torch.utils.data import DataLoader

from fms_acceleration_b200.compat import Accelerator
from fms_acceleration_b200.models.builder import build_model
from fms_acceleration_b200.plugins.odm import OnlineMixingDataset

UPDATE_EVERY = 10


class State:
    """Stand-in for a trainer state: the reward functions read ``log_history``."""

    def __init__(self):
        self.log_history = []
        self.global_step = 0


def make_category(vocab: int, lo: int, hi: int, n: int, length: int, seed: int):
    g = torch.Generator().manual_seed(seed)
    rows = []
    for _ in range(n):
        ids = torch.randint(lo, hi, (length,), generator=g)
        rows.append({"input_ids": ids, "attention_mask": torch.ones(length, dtype=torch.long), "labels": ids.clone()})
    return rows


def collate(rows):
    return {k: torch.stack([r[k] for r in rows]) for k in rows[0]}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--batch", type=int, default=4)
    a = ap.parse_args(argv)
    dev = torch.device(a.device)
    model = build_model("tiny-llama", device=dev, dtype=torch.float32 if dev.type == "cpu" else torch.bfloat16, seed=0)
    V = model.config.vocab_size
    # three "domains": disjoint token ranges, so their losses evolve differently
    train = {f"domain_{i}": make_category(V, i * 1000, (i + 1) * 1000, 64, 32, seed=i) for i in range(3)}
    evals = {k: make_category(V, i * 1000, (i + 1) * 1000, 8, 32, seed=100 + i) for i, k in enumerate(train)}
    out_dir = tempfile.mkdtemp(prefix="odm_")
    dataset = OnlineMixingDataset(train, {k: collate for k in train}, evals, {k: collate for k in evals},
                                  output_dir=out_dir, reward_type="entropy", sampling_interval=a.batch,
                                  eval_batch_size=4, vocab_size=V)
    # the dataset yields single samples (1-D tensors; labels as a list): stack them into a batch
    loader = DataLoader(dataset, batch_size=a.batch,
                        collate_fn=lambda rows: {k: torch.stack([torch.as_tensor(r[k]) for r in rows]) for k in rows[0]})
    accelerator = Accelerator(device=dev)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-4)
    state = State()
    model.train()
    for step, batch in enumerate(loader, start=1):
        if step > a.steps:
            break
        batch = {k: v.to(dev) for k, v in batch.items()}
        out = model(input_ids=batch["input_ids"], labels=batch["labels"])
        out.loss.backward()
        gn = torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        opt.step()
        opt.zero_grad(set_to_none=True)
        state.global_step = step
        state.log_history.append({"loss": float(out.loss.detach()), "grad_norm": float(gn), "step": step})
        if step % UPDATE_EVERY == 0:
            dataset.update_sampling_weights(model, accelerator, state)
            print(f"step {step}: loss {float(out.loss.detach()):.3f} sampling ratio "
                  f"{[round(r, 3) for r in dataset.sampling_ratio]}", flush=True)
    print(f"log: {dataset.log_file_path}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
