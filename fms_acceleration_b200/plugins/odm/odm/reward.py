"""Reward signals for the data-mixing bandit (semantics of fms_acceleration_odm/odm/reward.py:13-148).

* ``ENTROPY`` / ``ENTROPY3_VARENT1`` / ``ENTROPY_LAST_TOKEN``: run the model on an evaluation batch without gradients,
  take the per-token predictive entropy (and its variance), average over the attended positions of every sequence,
  normalise by ``log(vocab)`` (resp. its square), clamp to [0, 1] and sum over the batch.
* ``TRAIN_LOSS`` / ``VALIDATION_LOSS`` / ``GRADNORM``: per-category buffers fed from the trainer's log history; a
  high loss rewards a category, a high gradient norm penalises it (``1 / (gn + 1e-4)``).
"""
from __future__ import annotations

from enum import Enum
from typing import Dict, List, Optional

import torch
import torch.nn.functional as F


class Reward(str, Enum):
    ENTROPY = "entropy"
    ENTROPY3_VARENT1 = "entropy3_varent1"
    ENTROPY_LAST_TOKEN = "entropy_last_token"
    TRAIN_LOSS = "train_loss"
    VALIDATION_LOSS = "validation_loss"
    GRADNORM = "gradnorm"

    def __str__(self) -> str:
        return self.value

    @classmethod
    def parse(cls, v) -> "Reward":
        if isinstance(v, cls):
            return v
        s = str(v).lower()
        s = s.split(".")[-1]
        return cls(s)


# per-category memories of the history-based rewards (module level, as in the reference)
TRAIN_LOSS_DATA = {"buffer": []}
EVAL_LOSS_DATA = {"buffer": []}
GRADNORM_DATA = {"buffer": []}
_UNSEEN = 1e-100


def _entropy_stats(logits: torch.Tensor, attention_mask: torch.Tensor, vocab_size: int):
    shift = logits[:, :-1, :].float()
    logp = F.log_softmax(shift, dim=-1)
    p = logp.exp()
    ent = -(p * logp).sum(-1)
    varent = (p * logp.pow(2)).sum(-1) - ent.pow(2)
    last = ent[:, -1]
    m = attention_mask[:, 1:].to(ent.dtype)
    denom = m.sum(-1)
    ent = (ent * m).sum(-1) / denom
    varent = (varent * m).sum(-1) / denom
    hmax = torch.log(torch.tensor(float(vocab_size), dtype=ent.dtype, device=ent.device))
    return (ent / hmax).clamp(0, 1), (varent / hmax ** 2).clamp(0, 1), (last / hmax).clamp(0, 1)


def compute_reward(model, batch: Optional[Dict[str, torch.Tensor]], vocab_size: int, reward_type,
                   train_loss_history: Optional[List[dict]] = None, eval_loss_history: Optional[List[dict]] = None,
                   gradnorm_history: Optional[List[dict]] = None, last_sampled_category: Optional[int] = None,
                   total_categories: Optional[int] = None, current_category: Optional[int] = None) -> float:
    rt = Reward.parse(reward_type)
    if rt.value.startswith("entropy"):
        with torch.inference_mode():
            out = model(**batch)
            logits = out.logits if hasattr(out, "logits") else out["logits"]
            ent, varent, last = _entropy_stats(logits, batch["attention_mask"], vocab_size)
        if rt == Reward.ENTROPY:
            return ent.sum().item()
        if rt == Reward.ENTROPY3_VARENT1:
            return 0.75 * ent.sum().item() + 0.25 * varent.sum().item()
        return last.sum().item()
    if rt == Reward.TRAIN_LOSS:
        if not train_loss_history:
            raise ValueError("train_loss_history cannot be a empty list or None")
        if not TRAIN_LOSS_DATA["buffer"]:
            TRAIN_LOSS_DATA["buffer"] = [_UNSEEN] * total_categories
        TRAIN_LOSS_DATA["buffer"][last_sampled_category] = train_loss_history[-1]["loss"]
        return TRAIN_LOSS_DATA["buffer"][current_category]
    if rt == Reward.VALIDATION_LOSS:
        if not eval_loss_history:
            raise ValueError("eval_loss_history cannot be a empty list or None."
                             "Make sure you are using eval_strategy and eval_steps"
                             "allowing atleast 1 evaluation before reward computation.")
        if not EVAL_LOSS_DATA["buffer"]:
            EVAL_LOSS_DATA["buffer"] = [_UNSEEN] * total_categories
        EVAL_LOSS_DATA["buffer"][current_category] = eval_loss_history[-1]["loss"]
        return EVAL_LOSS_DATA["buffer"][current_category]
    if rt == Reward.GRADNORM:
        if not gradnorm_history:
            raise ValueError("gradnorm_history cannot be a empty list or None.Make sure grad norm is made available.")
        if not GRADNORM_DATA["buffer"]:
            GRADNORM_DATA["buffer"] = [_UNSEEN] * total_categories
        GRADNORM_DATA["buffer"][last_sampled_category] = 1.0 / (gradnorm_history[-1]["grad_norm"] + 0.0001)
        return GRADNORM_DATA["buffer"][current_category]
    raise TypeError(f"Reward {reward_type} not supported")
