"""Calibration-data helpers for GPTQ quantisation (role of fms_acceleration_peft/gptqmodel/utils/data.py)."""
from __future__ import annotations

from typing import Dict, List

import torch


def make_data_block(samples: Dict[str, List], prompt_col_name: str, label_col_name: str, tokenizer,
                    preprocess_fn=None, sample_max_len: int = 1024, block_max_len: int = 2048,
                    add_eos_token: bool = False, truncate_prompt: bool = True, merge_prompt_label: bool = False):
    """Tokenise prompt/label pairs and greedily merge short samples into blocks of at most ``block_max_len``."""
    if preprocess_fn:
        samples = preprocess_fn(samples)
    prompts, labels = samples[prompt_col_name], samples[label_col_name]
    tok_p = tokenizer(prompts, truncation=False)["input_ids"]
    tok_l = tokenizer(labels, truncation=False)["input_ids"]
    items = []
    for p, l in zip(tok_p, tok_l):
        if add_eos_token and getattr(tokenizer, "eos_token_id", None) is not None:
            l = l + [tokenizer.eos_token_id]
        if len(p) + len(l) > sample_max_len:
            if truncate_prompt:
                p = p[-max(sample_max_len - len(l), 0):] if sample_max_len > len(l) else []
                l = l[:sample_max_len]
            else:
                l = l[: max(sample_max_len - len(p), 0)]
        if len(p) + len(l) > 0:
            items.append((p, l))
    blocks, cur, cur_len = [], [], 0
    for p, l in sorted(items, key=lambda t: len(t[0]) + len(t[1])):
        n = len(p) + len(l)
        if cur and cur_len + n > block_max_len:
            blocks.append(cur)
            cur, cur_len = [], 0
        cur.append((p, l))
        cur_len += n
    if cur:
        blocks.append(cur)
    out = {"input_ids": [], "attention_mask": [], "labels": []}
    for blk in blocks:
        ids, lab = [], []
        for p, l in blk:
            ids += p + l
            lab += ([-100] * len(p) if not merge_prompt_label else p) + l
        out["input_ids"].append(ids)
        out["attention_mask"].append([1] * len(ids))
        out["labels"].append(lab)
    return out


def collate_data(blocks: List[Dict[str, List]], pad_token_id: int) -> Dict[str, torch.Tensor]:
    """Left-pad a list of examples to a rectangular batch."""
    def pad(rows, value):
        n = max(len(r) for r in rows)
        return torch.tensor([[value] * (n - len(r)) + list(r) for r in rows], dtype=torch.long)

    ids = [b["input_ids"] if not torch.is_tensor(b["input_ids"]) else b["input_ids"].reshape(-1).tolist() for b in blocks]
    am = [b.get("attention_mask", [1] * len(i)) for b, i in zip(blocks, ids)]
    am = [a if not torch.is_tensor(a) else a.reshape(-1).tolist() for a in am]
    out = {"input_ids": pad(ids, pad_token_id), "attention_mask": pad(am, 0)}
    if "labels" in blocks[0]:
        lab = [b["labels"] if not torch.is_tensor(b["labels"]) else b["labels"].reshape(-1).tolist() for b in blocks]
        out["labels"] = pad(lab, -100)
    return out


def get_dataloader(examples: List[Dict], batch_size: int = 1, pad_token_id: int = 0):
    """Batches of calibration examples (each ``{"input_ids": ..., "attention_mask": ...}``)."""
    return [collate_data(examples[i: i + batch_size], pad_token_id) for i in range(0, len(examples), batch_size)]
