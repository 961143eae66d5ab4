"""Helpers for sharded training of quantised models (cf. fms_acceleration_peft/fsdp_utils.py:27-98)."""
from __future__ import annotations

from collections import defaultdict
from typing import Callable, Optional

import torch


def ensure_weights_retied(param_init_fn: Optional[Callable], model: torch.nn.Module, device):
    """Wrap ``param_init_fn`` so that parameters that were tied before a module is re-materialised (e.g. the
    input and output embeddings) are tied again afterwards."""
    tied_groups = defaultdict(list)
    for name, p in model.named_parameters(remove_duplicate=False):
        tied_groups[id(p)].append(name)
    tied_groups = [names for names in tied_groups.values() if len(names) > 1]
    if not tied_groups:
        return param_init_fn

    owner_of = {}
    for names in tied_groups:
        for n in names:
            mod_name, _, pname = n.rpartition(".")
            owner_of[(model.get_submodule(mod_name) if mod_name else model, pname)] = tuple(names)
    materialised = {}

    def init_fn(module: torch.nn.Module):
        if param_init_fn is not None:
            param_init_fn(module)
        for (mod, pname), key in owner_of.items():
            if mod is not module:
                continue
            if key in materialised:
                setattr(module, pname, materialised[key])
            else:
                materialised[key] = getattr(module, pname)
        return module

    return init_fn


def put_selected_meta_tensors_on_cpu(model: torch.nn.Module) -> None:
    """Give the input / output embeddings real CPU storage when they are still on the meta device."""
    for getter in ("get_input_embeddings", "get_output_embeddings"):
        fn = getattr(model, getter, None)
        if fn is None:
            continue
        emb = fn()
        if emb is None:
            continue
        w = getattr(emb, "weight", None)
        if w is not None and w.is_meta:
            emb.weight = torch.nn.Parameter(torch.empty(*w.shape, dtype=w.dtype, device="cpu"),
                                            requires_grad=w.requires_grad)
