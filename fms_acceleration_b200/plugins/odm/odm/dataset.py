"""``OnlineMixingDataset``: an iterable dataset over K category datasets whose sampling ratios are learnt online with
the EXP3 multi-armed bandit.

Behaviour of fms_acceleration_odm/odm/dataset.py:24-562 in the reference:
  ratio_k  = (1 - gamma) * w_k / sum(w) + gamma / K
  update   : w_k *= exp(eta * (mean_reward_k / ratio_k) / K)
  sampling : every ``sampling_interval`` samples an arm is drawn from ``ratio`` with a dataset-local RNG seeded
             identically on all ranks; the arm's (stateful) loader yields the sample and restarts when exhausted
  logging  : one JSON line per sample / update in ``<output_dir>/odm_rank_<rank>.jsonl``
  resume   : ``state_dict`` / ``load_state_dict`` carry the bandit, the RNG states and every loader position
"""
from __future__ import annotations

import json
import math
import os
import random
from logging import getLogger
from typing import Any, Dict, List, Optional

import torch
from torch.utils.data import DataLoader, IterableDataset

from .auto_categorizer import AutoCategorizeConfig, DatasetAutoCategorizer
from .reward import Reward, compute_reward

logger = getLogger(__name__)


class _ResumableLoader:
    """Batch-size-1 sequential loader whose position can be saved and restored (the job ``StatefulDataLoader`` of
    torchdata does for the reference).  Map-style datasets are indexed; iterable (streaming) ones are consumed
    through their iterator and a restored position is reached by skipping that many samples."""

    def __init__(self, dataset, collate_fn=None):
        self.dataset, self.collate_fn = dataset, collate_fn
        self.streaming = isinstance(dataset, IterableDataset) or not hasattr(dataset, "__getitem__")
        self.pos = 0
        self._it = None

    def __iter__(self):
        self.pos = 0
        self._it = iter(self.dataset) if self.streaming else None
        return self

    def _next_item(self):
        if not self.streaming:
            if self.pos >= len(self.dataset):
                raise StopIteration
            return self.dataset[self.pos]
        if self._it is None:
            # first use, or a restored position: start the stream and skip what was already consumed
            self._it = iter(self.dataset)
            for _ in range(self.pos):
                next(self._it)
        return next(self._it)

    def __next__(self):
        item = self._next_item()
        self.pos += 1
        if self.collate_fn is not None:
            return self.collate_fn([item])
        return torch.utils.data.default_collate([item])

    def state_dict(self):
        return {"pos": self.pos}

    def load_state_dict(self, sd):
        self.pos = int(sd["pos"])
        self._it = None


class OnlineMixingDataset(IterableDataset):
    def __init__(self, dataset_dict: Dict[str, Any], collators_dict: Optional[dict], eval_dataset_dict: Dict[str, Any],
                 eval_collators_dict: Optional[dict], sampling_weights: Optional[dict] = None, gamma: float = 0.1,
                 eta: float = 0.3, sampling_interval: int = 1, eval_batch_size: int = 5, output_dir: str = "odm",
                 reward_type=Reward.ENTROPY, auto_categorize_config=None, seed: Optional[int] = 42,
                 vocab_size: int = 32000):
        self.auto_categorize = len(dataset_dict) == 1
        self._auto_categorize_config = self._build_auto_categorize_config(auto_categorize_config)
        dataset_dict, collators_dict = self._maybe_auto_categorize_dataset(dataset_dict, collators_dict, "train")
        eval_dataset_dict, eval_collators_dict = self._maybe_auto_categorize_dataset(
            eval_dataset_dict, eval_collators_dict, "eval")
        self.gamma, self.eta, self.sampling_interval = gamma, eta, sampling_interval
        self.collators_dict, self.eval_collators_dict = collators_dict, eval_collators_dict
        self.dataset_dict, self.eval_dataset_dict = dataset_dict, eval_dataset_dict
        self.eval_batch_size = eval_batch_size
        self.vocab_size = vocab_size
        self.train_dataset_dict_dl = {k: _ResumableLoader(v, collators_dict[k] if collators_dict else None)
                                      for k, v in dataset_dict.items()}
        self.train_dataset_dict_dl_iter = {k: iter(v) for k, v in self.train_dataset_dict_dl.items()}
        self.eval_dataset_dict_dl: Dict[str, Any] = {}
        self.category_list = sorted(self.train_dataset_dict_dl)
        self.id2cat = dict(enumerate(self.category_list))
        self.cat2id = {c: i for i, c in self.id2cat.items()}
        self.total_categories = len(self.category_list)
        self.rank = os.environ.get("RANK", "0")
        init = [1.0] * self.total_categories if not sampling_weights else [sampling_weights[c] for c in self.category_list]
        self.sampling_weights = torch.tensor(init, dtype=torch.float64)
        self.sampling_ratio: List[float] = []
        self._update_sampling_ratio(self.sampling_weights)
        self.curr_cat_count = [0] * self.total_categories
        self.produced = 0
        self.arm_idx = 0
        self.reward_type = Reward.parse(reward_type)
        self.output_dir = output_dir
        os.makedirs(output_dir, exist_ok=True)
        self.log_file_path = os.path.join(output_dir, f"odm_rank_{self.rank}.jsonl")
        self.log = {
            "samples_produced_so_far": 0, "sampling_interval": sampling_interval,
            "total_categories": self.total_categories, "current_sampling_weights": self.sampling_weights.tolist(),
            "current_sampling_ratio": self.sampling_ratio, "arm_idx": 0,
            "category_level_counts_so_far": self.curr_cat_count, "rewards": [0] * self.total_categories, "count": 0,
            "action": "", "rank": self.rank,
        }
        self.seed = 42 if seed is None else seed
        self._rng = random.Random(self.seed)
        self._current_epoch = 0
        self._rng_state_restored = False

    # ------------------------------------------------------------------ logging
    def log_to_file(self, data: dict) -> None:
        self.log.update(data)
        with open(self.log_file_path, "a", encoding="utf-8") as fh:
            fh.write(json.dumps(self.log) + "\n")

    # ------------------------------------------------------------------ iteration
    def __iter__(self):
        return self

    def set_epoch(self, epoch: int) -> None:
        """All ranks reseed identically per epoch (skipped once right after a restore)."""
        self._current_epoch = epoch
        if self._rng_state_restored:
            self._rng_state_restored = False
            return
        self._rng.seed(self.seed + epoch)

    def __next__(self):
        if self.produced % self.sampling_interval == 0:
            self.arm_idx = self._rng.choices(range(self.total_categories), weights=self.sampling_ratio, k=1)[0]
        cat = self.id2cat[self.arm_idx]
        try:
            sample = next(self.train_dataset_dict_dl_iter[cat])
        except StopIteration:
            logger.info("%s dataset exhausted so the iterator is reset.", cat)
            self.train_dataset_dict_dl_iter[cat] = iter(self.train_dataset_dict_dl[cat])
            sample = next(self.train_dataset_dict_dl_iter[cat])
        self.curr_cat_count[self.arm_idx] += 1
        self.produced += 1
        if isinstance(sample, torch.Tensor):
            ids = sample[0]
            sample = {"input_ids": ids, "attention_mask": torch.ones_like(ids), "labels": ids}
        else:
            ids = sample["input_ids"][0]
            sample = {
                "input_ids": ids,
                "attention_mask": sample["attention_mask"][0] if "attention_mask" in sample else torch.ones_like(ids),
                "labels": sample["labels"][0].tolist() if "labels" in sample else ids,
            }
        self.log_to_file({"arm_idx": self.arm_idx, "samples_produced_so_far": self.produced,
                          "category_level_counts_so_far": self.curr_cat_count, "action": "sample"})
        return sample

    # ------------------------------------------------------------------ checkpointing
    def state_dict(self) -> dict:
        return {
            "rng": torch.get_rng_state(), "gamma": self.gamma, "eta": self.eta,
            "sampling_interval": self.sampling_interval,
            "train_dataset_dict_dl_sd": {k: v.state_dict() for k, v in self.train_dataset_dict_dl_iter.items()},
            "eval_batch_size": self.eval_batch_size, "category_list": self.category_list, "id2cat": self.id2cat,
            "cat2id": self.cat2id, "total_categories": self.total_categories,
            "sampling_weights": self.sampling_weights, "sampling_ratio": self.sampling_ratio,
            "curr_cat_count": self.curr_cat_count, "produced": self.produced, "arm_idx": self.arm_idx,
            "reward_type": str(self.reward_type), "random_state": random.getstate(),
            "online_mixing_rng_state": self._rng.getstate(), "seed": self.seed, "_current_epoch": self._current_epoch,
        }

    def load_state_dict(self, state_dict: dict) -> None:
        sd = dict(state_dict)
        torch.set_rng_state(sd["rng"])
        loaders = sd.pop("train_dataset_dict_dl_sd")
        random.setstate(sd.pop("random_state"))
        rng_state = sd.pop("online_mixing_rng_state", None)
        seed = sd.pop("seed", None)
        epoch = sd.pop("_current_epoch", None)
        if seed is not None:
            self.seed = seed
        if epoch is not None:
            self._current_epoch = epoch
        if rng_state is not None:
            self._rng.setstate(rng_state)
            self._rng_state_restored = True
        for k, v in sd.items():
            if k not in ("rng", "reward_type") and hasattr(self, k):
                setattr(self, k, v)
        self.reward_type = Reward.parse(sd["reward_type"])
        for k, v in loaders.items():
            self.train_dataset_dict_dl_iter[k].load_state_dict(v)

    # ------------------------------------------------------------------ auto categorisation
    def _build_auto_categorize_config(self, config):
        if isinstance(config, AutoCategorizeConfig):
            return config
        return AutoCategorizeConfig() if config is None else AutoCategorizeConfig(**config)

    def _maybe_auto_categorize_dataset(self, container, collators_dict, dataset_role):
        if len(container) != 1:
            return container, collators_dict
        candidate = next(iter(container.values()))
        categorised = DatasetAutoCategorizer(config=self._auto_categorize_config)(dataset=candidate)
        collators_dict = self._broadcast_collators_to_auto_categories(collators_dict, list(categorised.keys()))
        logger.info("Auto-categorized %s dataset into %d pseudo categories", dataset_role, len(categorised))
        return categorised, collators_dict

    def _broadcast_collators_to_auto_categories(self, collators_dict, category_names):
        if not category_names:
            return collators_dict or {}
        if not collators_dict:
            return {n: None for n in category_names}
        if set(collators_dict) == set(category_names):
            return dict(collators_dict)
        if len(collators_dict) == 1:
            only = next(iter(collators_dict.values()))
            return {n: only for n in category_names}
        raise ValueError("Unable to broadcast collators to auto-categorized datasets. Provide a single "
                         "collator or one entry per generated category.")

    # ------------------------------------------------------------------ EXP3
    def _update_sampling_ratio(self, weights) -> list:
        K = len(weights)
        self.sampling_ratio = ((1.0 - self.gamma) * (weights / weights.sum()) + self.gamma / K).tolist()
        return self.sampling_ratio

    def _update_weights(self, count, rewards) -> list:
        for arm in range(self.total_categories):
            mean_r = float(rewards[arm]) / float(count[arm])
            estimate = mean_r / self.sampling_ratio[arm]
            self.sampling_weights[arm] *= math.exp(self.eta * estimate / self.total_categories)
        return self._update_sampling_ratio(self.sampling_weights)

    def _extract_information_from_state_for_reward(self, state=None, category=None) -> dict:
        if state is None or self.reward_type.value.startswith("entropy"):
            return {}
        hist = state.log_history
        if self.reward_type == Reward.TRAIN_LOSS:
            return {"train_loss_history": [d for d in hist if "loss" in d]}
        if self.reward_type == Reward.VALIDATION_LOSS:
            assert category is not None
            key = f"eval_{category}_loss"
            return {"eval_loss_history": [{"loss": d[key], **d} for d in hist if key in d]}
        if self.reward_type == Reward.GRADNORM:
            return {"gradnorm_history": [d for d in hist if "grad_norm" in d]}
        return {}

    def _reset_eval_dataloaders(self) -> None:
        self.eval_dataset_dict_dl = {}
        for k, ds in self.eval_dataset_dict.items():
            self.eval_dataset_dict_dl[k] = iter(DataLoader(
                ds, self.eval_batch_size, shuffle=True, num_workers=0,
                collate_fn=self.eval_collators_dict[k] if self.eval_collators_dict else None)) if ds else None

    def update_sampling_weights(self, model, accelerator, state) -> None:
        """One bandit update: reward of every category (over its evaluation set for the entropy rewards, from the
        trainer history otherwise), summed over ranks, then the EXP3 weight update."""
        rewards = [0.0] * self.total_categories
        count = [0] * self.total_categories
        device = accelerator.device if accelerator else (
            torch.device("cuda", 0) if torch.cuda.is_available() else torch.device("cpu"))
        self._reset_eval_dataloaders()
        for c in range(self.total_categories):
            cat = self.id2cat[c]
            loader = self.eval_dataset_dict_dl.get(cat)
            if loader is not None and accelerator is not None:
                loader = accelerator.prepare(loader)
            extra = self._extract_information_from_state_for_reward(state, cat)
            common = dict(model=model, vocab_size=self.vocab_size, reward_type=self.reward_type, current_category=c,
                          total_categories=self.total_categories, last_sampled_category=self.arm_idx, **extra)
            if not loader:
                rewards[c] += compute_reward(batch=None, **common)
                count[c] += 1
                continue
            for batch in loader:
                rewards[c] += compute_reward(batch={k: v.to(device) for k, v in batch.items()}, **common)
                count[c] += batch["input_ids"].shape[0]
        rewards_t = torch.tensor(rewards, device=device, dtype=torch.float64 if device.type == "cpu" else torch.float32)
        count_t = torch.tensor(count, device=device)
        if accelerator:
            rewards_t = accelerator.reduce(rewards_t, reduction="sum")
            count_t = accelerator.reduce(count_t, reduction="sum")
        self._update_weights(count_t, rewards_t)
        self.log_to_file({"current_sampling_weights": self.sampling_weights.tolist(),
                          "current_sampling_ratio": self.sampling_ratio, "rewards": rewards_t.tolist(),
                          "count": count_t.tolist(), "action": "update"})
