"""Mapping between Hugging Face MoE checkpoints and ScatterMoE parameters.

Two checkpoint styles exist (fms_acceleration_moe/utils/scattermoe_state_dict.py:82-338 of the reference):
*sharded* (Mixtral: ``experts.<i>.w1.weight`` ``[out, in]`` per expert) and *fused* (GraniteMoe:
``input_linear.weight [E, 2I, H]`` whose first ``I`` rows are ``w1`` and last ``I`` rows ``w3``,
``output_linear.weight [E, H, I]``).  ScatterMoE keeps ``w{1,2,3}.weight`` as ``[E, in, out]`` and the router as
``router.weight [E, H]``.
"""
from __future__ import annotations

import json
import os
import re
from collections import OrderedDict, defaultdict
from typing import Dict, List, Optional, Tuple

import torch

from .scattermoe_constants import (DIM_EXPERT, FILE_SAFETENSOR_INDEX, KEY_SCATTERMOE_ROUTER,
                                   PARAM_NAME_WEIGHT_SCATTERMOE)


def _set_at(lst: List, i: int, v) -> None:
    while len(lst) <= i:
        lst.append(None)
    lst[i] = v


def _expert_map_from_name(expert_name: str) -> Dict[str, List[str]]:
    if "|" not in expert_name:
        return {w: [w] for w in PARAM_NAME_WEIGHT_SCATTERMOE}
    names = expert_name.split("|")
    limit = len(PARAM_NAME_WEIGHT_SCATTERMOE)
    assert 2 <= len(names) <= limit, f"If expert_name has |, expect between 2 and {limit} entries, but got {len(names)}."
    mapping: Dict[str, List[str]] = {}
    for i, n in enumerate(names):
        mapping.setdefault(n, []).append(PARAM_NAME_WEIGHT_SCATTERMOE[i])
    return mapping


def get_checkpoint_meta_from_sharded_safetensor(weight_map: Dict, prefix: str, instance_name: str,
                                                router_name: str = "gate", expert_name: str = "experts",
                                                expert_map: Optional[Dict] = None) -> Dict[str, List[Tuple]]:
    """``{"router.weight": [(ckpt_key, file)], "w1.weight": [(key, file), ...per expert or one fused...], ...}`` for
    the MoE block ``<prefix>.<instance_name>``."""
    if expert_map is None:
        expert_map = _expert_map_from_name(expert_name)
    out: Dict[str, List] = defaultdict(list)
    full_prefix = f"{prefix}.{instance_name}."
    pattern = re.compile(rf"({router_name}|{expert_name})\.?(\d+)?\.?(\w+)?\.weight")
    # transformers >= 5 stores a per-expert-linear family (Mixtral) as two fused 3-D parameters without ".weight":
    # "<experts>.gate_up_proj" [E, 2I, H] (gate rows first) and "<experts>.down_proj" [E, H, I]
    fused3d = {"gate_up_proj": ["w1", "w3"], "down_proj": ["w2"]}
    for key, st_file in weight_map.items():
        if not key.startswith(full_prefix):
            continue
        rel = key[len(full_prefix):]
        head, _, tail = rel.rpartition(".")
        if head == expert_name.split("|")[0] and tail in fused3d:
            for w in fused3d[tail]:
                _set_at(out[f"{w}.weight"], 0, (key, st_file))
            continue
        m = pattern.match(rel)
        if m is None:
            raise ValueError(
                f"Unable to handle key '{key}' with provided router_name '{router_name}' or expert_name '{expert_name}'")
        if m.group(1) == router_name:
            out[KEY_SCATTERMOE_ROUTER].append((key, st_file))
            continue
        index = int(m.group(2)) if m.group(2) is not None else 0
        targets = expert_map.get(m.group(1), expert_map.get(m.group(3)))
        assert targets, f"cannot map '{rel}'"
        for w in targets:
            _set_at(out[f"{w}.weight"], index, (key, st_file))
    if len(out) == 0:
        raise ValueError(f"Could not get safetensor map for '{full_prefix}' and '{instance_name}'")
    return out


def _maybe_reshape_scattermoe_expert_weights(weights: torch.Tensor, scatter_key: str, intermediate_size: int,
                                             num_experts: Optional[int] = None) -> torch.Tensor:
    """Checkpoint expert tensor ([E?, out, in], possibly fused gate|up rows) -> ScatterMoE ``[E, in, out]``."""
    if weights.dim() == 2:
        weights = weights.unsqueeze(0) if num_experts in (None, 1) else weights.view(num_experts, -1, weights.shape[-1])
    name = scatter_key.split(".")[0]
    if name in ("w1", "w3") and weights.shape[1] == 2 * intermediate_size:
        weights = weights[:, :intermediate_size] if name == "w1" else weights[:, intermediate_size:]
    return weights.permute(0, 2, 1).contiguous()


def convert_state_dict(prefix: str, checkpoint_metadata: Dict[str, List[Tuple]], state_dict: Dict[str, torch.Tensor],
                       num_experts: int, intermediate_size: int, dtype: Optional[torch.dtype] = None) -> "OrderedDict":
    """In-memory conversion of one MoE block (state dict already loaded)."""
    target = OrderedDict()
    for scatter_key, entries in checkpoint_metadata.items():
        tensors = [state_dict[k if k in state_dict else k[len(prefix):]] for k, _ in entries]
        if scatter_key == KEY_SCATTERMOE_ROUTER:
            t = tensors[0]
        else:
            t = tensors[0] if len(tensors) == 1 else torch.stack(tensors, dim=DIM_EXPERT)
            t = _maybe_reshape_scattermoe_expert_weights(t, scatter_key, intermediate_size, num_experts)
        target[scatter_key] = t.to(dtype) if dtype is not None else t
    return target


def get_state_dict_from_checkpoint_metadata(checkpoint_directory: str, checkpoint_metadata: Dict[str, List[Tuple]],
                                            num_experts: int, intermediate_size: int, expert_start: int = 0,
                                            expert_end: Optional[int] = None, dtype: Optional[torch.dtype] = None):
    """Read only the experts ``[expert_start, expert_end)`` of one MoE block from safetensors files."""
    from safetensors import safe_open

    expert_end = num_experts if expert_end is None else expert_end
    handles = {}

    def _open(fname):
        if fname not in handles:
            handles[fname] = safe_open(os.path.join(checkpoint_directory, fname), framework="pt")
        return handles[fname]

    target = OrderedDict()
    for scatter_key, entries in checkpoint_metadata.items():
        if scatter_key == KEY_SCATTERMOE_ROUTER:
            k, f = entries[0]
            t = _open(f).get_tensor(k)
        elif len(entries) == 1:  # fused [E, out, in]
            k, f = entries[0]
            t = _open(f).get_slice(k)[expert_start:expert_end]
            t = _maybe_reshape_scattermoe_expert_weights(t, scatter_key, intermediate_size)
        else:  # one tensor per expert
            parts = [_open(f).get_tensor(k) for k, f in entries[expert_start:expert_end]]
            t = _maybe_reshape_scattermoe_expert_weights(torch.stack(parts, dim=DIM_EXPERT), scatter_key, intermediate_size)
        target[scatter_key] = t.to(dtype) if dtype is not None else t
    return target


def load_weight_map(checkpoint_directory: str) -> Dict[str, str]:
    """Key -> safetensors file of a (sharded or single-file) checkpoint."""
    index = os.path.join(checkpoint_directory, FILE_SAFETENSOR_INDEX)
    if os.path.exists(index):
        with open(index, encoding="utf-8") as fh:
            return json.load(fh)["weight_map"]
    single = os.path.join(checkpoint_directory, "model.safetensors")
    if os.path.exists(single):
        from safetensors import safe_open

        with safe_open(single, framework="pt") as f:
            return {k: "model.safetensors" for k in f.keys()}
    raise FileNotFoundError(f"no safetensors checkpoint in {checkpoint_directory}")
