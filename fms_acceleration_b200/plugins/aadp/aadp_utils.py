"""Collators and helpers for padding-free training (role of fms_acceleration_aadp/aadp_utils.py:25-89)."""
from __future__ import annotations

from types import MethodType
from typing import Any, Dict, List

import numpy as np
import torch


class DataCollatorWithFlattening:
    """Concatenate a mini-batch into one ``[1, total_tokens]`` row without padding.

    Returns ``input_ids``, ``labels`` and ``position_ids``; positions restart at 0 for every sample and the
    first label of every sample is ``-100`` so that no token is predicted across a document boundary.
    Anything else in the features is dropped.
    """

    def __init__(self, return_tensors: str = "pt", return_cu_seqlens: bool = False):
        self.return_tensors = return_tensors
        self.return_cu_seqlens = return_cu_seqlens

    def __call__(self, features: List[Dict[str, Any]], return_tensors=None) -> Dict[str, torch.Tensor]:
        has_labels = "labels" in features[0]
        ids: List[int] = []
        labels: List[int] = []
        pos: List[int] = []
        cu = [0]
        for f in features:
            x = list(f["input_ids"]) if not torch.is_tensor(f["input_ids"]) else f["input_ids"].reshape(-1).tolist()
            ids += x
            pos += list(range(len(x)))
            src = x if not has_labels else (
                list(f["labels"]) if not torch.is_tensor(f["labels"]) else f["labels"].reshape(-1).tolist())
            labels += [-100] + src[1:]
            cu.append(cu[-1] + len(x))
        out = {
            "input_ids": torch.tensor([ids], dtype=torch.long),
            "labels": torch.tensor([labels], dtype=torch.long),
            "position_ids": torch.tensor([pos], dtype=torch.long),
        }
        if self.return_cu_seqlens:
            out["cu_seqlens"] = torch.tensor(cu, dtype=torch.int32)
        return out


def patch_torch_call_remove_padding(collate_fn):
    """Wrap a padding collator's ``torch_call`` so that pad positions are dropped and the batch is flattened."""
    original = collate_fn.torch_call

    def _torch_call(self, examples):
        batch = original(examples)
        mask = batch.pop("attention_mask").bool()
        batch["input_ids"] = batch["input_ids"][mask].unsqueeze(0)
        batch["position_ids"] = (mask.long().cumsum(1))[mask].unsqueeze(0) - 1
        batch["labels"] = batch["labels"][mask].unsqueeze(0)
        batch["labels"][batch["position_ids"] == 0] = getattr(self, "ignore_index", -100)
        return batch

    collate_fn.torch_call = MethodType(_torch_call, collate_fn)
    return collate_fn


def calculate_token_lengths(dataset, num_processes: int = 1) -> np.ndarray:
    """Token count of every sample.  Uses ``datasets.Dataset.map`` when available, else a plain loop."""
    if hasattr(dataset, "map") and hasattr(dataset, "column_names"):
        mapped = dataset.map(lambda x: {"len": len(x["input_ids"])}, num_proc=num_processes, load_from_cache_file=True)
        return np.array(mapped["len"])
    return np.array([len(dataset[i]["input_ids"]) for i in range(len(dataset))], dtype=np.int64)
