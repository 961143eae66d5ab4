"""Sharded checkpoints for ScatterMoE training and their conversion back to Hugging Face safetensors.

Directory contract (fms_acceleration_moe/utils/checkpoint_utils.py:72-771 of the reference): a checkpoint directory
holds ``pytorch_model_fsdp_<i>/`` with the model state saved by ``torch.distributed.checkpoint`` under the key
``"model"`` and ``optimizer_<i>/`` with the optimizer state under ``"optimizer"``; LoRA runs store only the
``lora_A`` / ``lora_B`` tensors (router adapters excluded).  ``recover_safetensors_from_dcp`` (also the module's
command line: ``python -m ...checkpoint_utils <dcp_dir> <out_dir> <pretrained_name>``) loads such a checkpoint
without a process group, strips the PEFT prefixes, maps ScatterMoE parameters (``router`` / ``w1`` / ``w2`` /
``w3`` ``[E, in, out]``) back to the original layout (per-expert linears or fused ``input_linear``) and writes
safetensors shards with an index.
"""
from __future__ import annotations

import json
import os
import re
import sys
from collections import defaultdict
from typing import Dict, List, Optional

import torch

from .scattermoe_constants import (FILE_SAFETENSOR_INDEX, PARAM_NAME_ROUTER_SCATTERMOE, PARAM_NAME_WEIGHT_SCATTERMOE,
                                   get_scattermoe_conv_spec_from_archs)
from .scattermoe_state_dict import get_checkpoint_meta_from_sharded_safetensor, load_weight_map

FSDP_MODEL_NAME = "pytorch_model_fsdp"
OPTIMIZER_NAME = "optimizer"
KEY_MODEL = "model"
KEY_OPTIMIZER = "optimizer"
SAFE_WEIGHTS_NAME = "model.safetensors"
ADAPTER_SAFE_WEIGHTS_NAME = "adapter_model.safetensors"
MODEL_INDEX = None  # index of the model within accelerate's model list, recorded by the save hook


# ------------------------------------------------------------------------------------------- save / load
# Expert parallelism: every rank holds the experts [rank * E/ep, (rank + 1) * E/ep) as an ordinary tensor under the
# SAME name.  Written as such, the checkpoint writer would treat them as replicas and keep one rank's copy.  They
# are therefore presented to torch.distributed.checkpoint as DTensors sharded on dim 0 over the expert-parallel
# group (what the reference's parameters are in the first place, scattermoe_prepare.py:64-99): every shard is
# written with its offset, a reader without a process group sees the full [E, in, out] tensor, and a reader with
# the same layout gets its own shard back.  AdamW moments of those parameters are wrapped the same way.
_MESHES: dict = {}


def _ep_mesh(group, device_type: str):
    from torch.distributed.device_mesh import DeviceMesh

    key = (id(group), device_type)
    if key not in _MESHES:
        _MESHES[key] = DeviceMesh.from_group(group, device_type)
    return _MESHES[key]


def _as_sharded(t: torch.Tensor, group):
    """Local expert shard -> DTensor Shard(0) over the expert-parallel group (shares storage with ``t``)."""
    from torch.distributed.tensor import DTensor, Shard

    return DTensor.from_local(t.detach(), _ep_mesh(group, t.device.type), [Shard(0)], run_check=False)


def _ep_param_names(model: torch.nn.Module) -> Dict[str, object]:
    """name -> expert-parallel group of every parameter sharded over experts."""
    out = {}
    if not (torch.distributed.is_available() and torch.distributed.is_initialized()):
        return out
    for n, p in model.named_parameters():
        g = getattr(p, "_fmsb_ep_group", None)
        if getattr(p, "_fmsb_expert_parallel", False) and g is not None and torch.distributed.get_world_size(g) > 1:
            out[n] = g
    return out


def _model_state(model: torch.nn.Module, lora_only: bool) -> Dict[str, torch.Tensor]:
    sd = model.state_dict()
    if lora_only:
        sd = {k: v for k, v in sd.items() if ("lora_A" in k or "lora_B" in k) and "router" not in k}
    for n, g in _ep_param_names(model).items():
        if n in sd:
            sd[n] = _as_sharded(sd[n], g)
    return sd


def _unwrap_state(sd: Dict) -> Dict:
    from torch.distributed.tensor import DTensor

    return {k: (v.to_local() if isinstance(v, DTensor) else v) for k, v in sd.items()}


def _optimizer_state(optimizer, model: torch.nn.Module) -> Dict:
    """``optimizer.state_dict()`` with the moments of expert-parallel parameters wrapped as sharded DTensors."""
    osd = optimizer.state_dict()
    ep = _ep_param_names(model)
    if not ep or not hasattr(optimizer, "param_groups"):
        return osd
    by_id = {id(p): n for n, p in model.named_parameters()}
    idx = 0
    for g in optimizer.param_groups:
        for p in g["params"]:
            name = by_id.get(id(p))
            st = osd["state"].get(idx)
            if name in ep and st is not None:
                st = dict(st)  # the optimizer hands out its live per-parameter dict: wrap in a copy
                osd["state"][idx] = st
                for k, v in list(st.items()):
                    if torch.is_tensor(v) and v.dim() > 0 and v.shape == p.shape:
                        st[k] = _as_sharded(v, ep[name])
            idx += 1
    return osd


def _unwrap_optimizer_state(osd: Dict) -> Dict:
    from torch.distributed.tensor import DTensor

    for idx, st in list(osd.get("state", {}).items()):
        if any(isinstance(v, DTensor) for v in st.values()):
            osd["state"][idx] = {k: (v.to_local() if isinstance(v, DTensor) else v) for k, v in st.items()}
    return osd


def save_fsdp_model(fsdp_plugin, accelerator, model: torch.nn.Module, output_dir: str, model_index: int = 0, **kwargs):
    """Model weights are written together with the optimizer (``save_fsdp_optimizer``); only remember the index."""
    global MODEL_INDEX
    MODEL_INDEX = model_index


def save_fsdp_optimizer(fsdp_plugin, accelerator, optimizer, model: torch.nn.Module, output_dir: str,
                        optimizer_index: int = 0, lora_only: Optional[bool] = None):
    import torch.distributed.checkpoint as dcp

    if fsdp_plugin is not None and getattr(fsdp_plugin, "state_dict_type", "SHARDED_STATE_DICT") not in (
            "SHARDED_STATE_DICT", None) and "SHARDED" not in str(fsdp_plugin.state_dict_type):
        raise NotImplementedError("Checkpointing for megablocks only enabled for sharded state dict.")
    if lora_only is None:
        lora_only = any("lora_" in n for n, _ in model.named_parameters())
    midx = MODEL_INDEX if MODEL_INDEX is not None else 0
    model_dir = os.path.join(output_dir, f"{FSDP_MODEL_NAME}_{midx}")
    opt_dir = os.path.join(output_dir, f"{OPTIMIZER_NAME}_{optimizer_index}")
    os.makedirs(model_dir, exist_ok=True)
    os.makedirs(opt_dir, exist_ok=True)
    no_dist = not (torch.distributed.is_available() and torch.distributed.is_initialized())
    dcp.save({KEY_MODEL: _model_state(model, lora_only)}, storage_writer=dcp.FileSystemWriter(model_dir), no_dist=no_dist)
    osd = optimizer.sharded_state_dict() if hasattr(optimizer, "sharded_state_dict") else _optimizer_state(optimizer, model)
    dcp.save({KEY_OPTIMIZER: osd}, storage_writer=dcp.FileSystemWriter(opt_dir), no_dist=no_dist)


def load_fsdp_model(fsdp_plugin, accelerator, model: torch.nn.Module, input_dir: str, model_index: int = 0, **kwargs):
    global MODEL_INDEX
    MODEL_INDEX = model_index


def _materialize_optimizer_state(optimizer) -> None:
    """A fresh optimizer has no per-parameter state, and a template without those entries makes the checkpoint
    reader skip them.  Create them with one step at learning rate 0 on zero gradients (parameters are unchanged)."""
    if len(optimizer.state) > 0:
        return
    saved = [g["lr"] for g in optimizer.param_groups]
    touched = []
    for g in optimizer.param_groups:
        g["lr"] = 0.0 if not torch.is_tensor(g["lr"]) else torch.zeros_like(g["lr"])
        for p in g["params"]:
            if p.requires_grad and p.grad is None:
                p.grad = torch.zeros_like(p)
                touched.append(p)
    optimizer.step()
    for p in touched:
        p.grad = None
    for g, lr in zip(optimizer.param_groups, saved):
        g["lr"] = lr


def load_fsdp_optimizer(fsdp_plugin, accelerator, optimizer, model: torch.nn.Module, input_dir: str,
                        optimizer_index: int = 0, lora_only: Optional[bool] = None):
    import torch.distributed.checkpoint as dcp

    if accelerator is not None:
        accelerator.wait_for_everyone()
    if lora_only is None:
        lora_only = any("lora_" in n for n, _ in model.named_parameters())
    midx = MODEL_INDEX if MODEL_INDEX is not None else 0
    no_dist = not (torch.distributed.is_available() and torch.distributed.is_initialized())
    msd = {KEY_MODEL: _model_state(model, lora_only)}
    dcp.load(msd, storage_reader=dcp.FileSystemReader(os.path.join(input_dir, f"{FSDP_MODEL_NAME}_{midx}")), no_dist=no_dist)
    model.load_state_dict(_unwrap_state(msd[KEY_MODEL]), strict=not lora_only)
    opt_dir = os.path.join(input_dir, f"{OPTIMIZER_NAME}_{optimizer_index}")
    if hasattr(optimizer, "load_sharded_state_dict"):
        # optimizer states sharded over the ranks: every rank reads its own slice of the flat state
        osd = {KEY_OPTIMIZER: optimizer.sharded_state_dict()}
        dcp.load(osd, storage_reader=dcp.FileSystemReader(opt_dir), no_dist=no_dist)
        optimizer.load_sharded_state_dict(osd[KEY_OPTIMIZER])
        return
    _materialize_optimizer_state(optimizer)
    osd = {KEY_OPTIMIZER: _optimizer_state(optimizer, model)}
    dcp.load(osd, storage_reader=dcp.FileSystemReader(opt_dir), no_dist=no_dist)
    optimizer.load_state_dict(_unwrap_optimizer_state(osd[KEY_OPTIMIZER]))


def patch_huggingface_save_and_load_for_dtensors() -> bool:
    """Point ``transformers.trainer``'s FSDP save / load helpers at the functions above (when transformers is there)."""
    try:
        import transformers.trainer as tr
    except Exception:
        return False
    for name, fn in (("save_fsdp_model", save_fsdp_model), ("save_fsdp_optimizer", save_fsdp_optimizer),
                     ("load_fsdp_model", load_fsdp_model), ("load_fsdp_optimizer", load_fsdp_optimizer)):
        if hasattr(tr, name):
            setattr(tr, name, fn)
    return True


def patch_huggingface_clip_grad_norm_fsdp2(accelerator) -> None:
    """Give the accelerator the expert-parallel aware gradient clipping."""
    accelerator.clip_grad_norm_ = lambda parameters, max_norm, norm_type=2.0: clip_grad_norm_(parameters, max_norm, norm_type)


def patch_prepare_sd_options() -> bool:
    """The reference replaces accelerate's ``_prepare_sd_options`` so that FSDP2 writes sharded state dicts that
    include the ScatterMoE DTensors (fms_acceleration_moe/utils/checkpoint_utils.py:161-180).  Checkpoints here are
    written by :func:`save_fsdp_model` / :func:`save_fsdp_optimizer` without FSDP, so there is nothing to prepare;
    the function exists for callers of the reference's name and reports whether accelerate is importable."""
    try:
        import accelerate.utils.fsdp_utils  # noqa: F401
    except Exception:
        return False
    return True


def patch_huggingface_fsdp2_load_full_state_dict() -> bool:
    """Counterpart of the reference's patch of ``fsdp2_load_full_state_dict`` / ``fsdp2_prepare_model``
    (:775-1037), which teaches accelerate's rank-0 loading to skip the already-placed expert shards.  Expert shards
    are read per rank straight from the safetensors files in ``prepare_scattermoe`` and no FSDP2 wrapper is
    involved, so no patch is applied; returns whether accelerate is importable."""
    return patch_prepare_sd_options()


def fsdp2_load_full_state_dict(accelerator, model: torch.nn.Module, full_sd: Optional[dict]) -> torch.nn.Module:
    """Load a FULL state dict that only rank 0 needs to hold into the model of every rank (the job of the reference's
    function of this name, :775-880, for FSDP2-sharded models).  Here ordinary parameters are replicated and expert
    tensors hold ``E / ep`` experts of the group: rank 0 broadcasts every tensor, a rank copies what it owns (its
    slice of dimension 0 for expert-parallel parameters).  Without a process group the dict is simply loaded."""
    dist = torch.distributed
    multi = dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1
    ep_groups = _ep_param_names(model)
    own = dict(model.named_parameters())
    own.update(dict(model.named_buffers()))
    names = sorted(own)
    if multi:
        holder = [sorted(k for k in (full_sd or {}) if k in own)] if dist.get_rank() == 0 else [None]
        dist.broadcast_object_list(holder, src=0)
        names = holder[0]
    elif full_sd is not None:
        names = [k for k in names if k in full_sd]
    with torch.no_grad():
        for name in names:
            dst = own[name]
            g = ep_groups.get(name)
            rows = dst.shape[0] * (dist.get_world_size(g) if g is not None else 1) if dst.dim() else 0
            full_shape = (rows,) + tuple(dst.shape[1:]) if dst.dim() else ()
            if multi:
                buf = (full_sd[name].to(device=dst.device, dtype=dst.dtype).contiguous() if dist.get_rank() == 0
                       else torch.empty(full_shape, device=dst.device, dtype=dst.dtype))
                dist.broadcast(buf, src=0)
            else:
                buf = full_sd[name].to(device=dst.device, dtype=dst.dtype)
            if g is not None and buf.shape[0] != dst.shape[0]:
                r = dist.get_rank(g)
                buf = buf[r * dst.shape[0]:(r + 1) * dst.shape[0]]
            dst.copy_(buf)
    return model


def fsdp2_prepare_model(accelerator, model: torch.nn.Module) -> torch.nn.Module:
    """Make the model ready for sharded multi-GPU training and hand it back (the reference wraps it with FSDP2 here,
    :883-1037).  This package shards through its own engine (frozen packed weights, gradient bucket, optimizer
    state); with one process the model is returned as it is."""
    from ....parallel.engine import install_engine

    if accelerator is not None and next(model.parameters()).is_cuda:
        install_engine(model, accelerator)
    return model


def clip_grad_norm_(parameters, max_norm: float, norm_type: float = 2.0, foreach=None) -> torch.Tensor:
    """Total gradient norm over replicated AND expert-parallel parameters: the squared norms of expert shards are
    summed over their expert-parallel group before the global norm is formed (the reference's FSDP2 version,
    checkpoint_utils.py:690-731, gathers DTensor norms the same way)."""
    params = [p for p in parameters if p.grad is not None]
    if not params:
        return torch.tensor(0.0)
    dev = params[0].grad.device
    rep = [p for p in params if not getattr(p, "_fmsb_expert_parallel", False)]
    exp = [p for p in params if getattr(p, "_fmsb_expert_parallel", False)]

    def _pow_sum(ps):
        if not ps:
            return torch.zeros((), device=dev)
        return torch.stack([p.grad.float().norm(norm_type) ** norm_type for p in ps]).sum()

    total = _pow_sum(rep)
    e = _pow_sum(exp)
    if exp and torch.distributed.is_available() and torch.distributed.is_initialized():
        torch.distributed.all_reduce(e)  # expert shards are disjoint across the expert-parallel ranks
        n_rep = max(torch.distributed.get_world_size() // max(_ep_size(exp[0]), 1), 1)
        e = e / n_rep
    norm = (total + e) ** (1.0 / norm_type)
    coef = (max_norm / (norm + 1e-6)).clamp(max=1.0)
    for p in params:
        p.grad.mul_(coef.to(p.grad.dtype))
    return norm


def _ep_size(p) -> int:
    g = getattr(p, "_fmsb_replicate_group", None)
    if g is None or not torch.distributed.is_initialized():
        return torch.distributed.get_world_size() if torch.distributed.is_initialized() else 1
    return torch.distributed.get_world_size() // torch.distributed.get_world_size(g)


# ------------------------------------------------------------------------------------------- readers
def get_state_dict_from_dcp_checkpoint(dcp_checkpoint_dir: str) -> Dict[str, torch.Tensor]:
    """Load a DCP checkpoint into plain tensors without a process group."""
    from torch.distributed.checkpoint.default_planner import _EmptyStateDictLoadPlanner
    from torch.distributed.checkpoint.state_dict_loader import _load_state_dict
    import torch.distributed.checkpoint as dcp

    sd: Dict = {}
    _load_state_dict(sd, storage_reader=dcp.FileSystemReader(dcp_checkpoint_dir), planner=_EmptyStateDictLoadPlanner(),
                     no_dist=True)
    return sd[KEY_MODEL] if KEY_MODEL in sd else sd


def get_state_dict_from_safe_checkpoint(safe_checkpoint_dir: str) -> Dict[str, torch.Tensor]:
    from safetensors import safe_open

    sd = {}
    for fname in sorted(set(load_weight_map(safe_checkpoint_dir).values())):
        with safe_open(os.path.join(safe_checkpoint_dir, fname), framework="pt") as f:
            for k in f.keys():
                sd[k] = f.get_tensor(k)
    return sd


def get_resolved_checkpoint_location(pretrained_model_name_or_path: str) -> str:
    """A local directory is its own location (there is no hub access in this environment)."""
    if os.path.isdir(pretrained_model_name_or_path):
        return pretrained_model_name_or_path
    raise FileNotFoundError(f"'{pretrained_model_name_or_path}' is not a local checkpoint directory")


def _read_architectures(pretrained_dir: str) -> List[str]:
    with open(os.path.join(pretrained_dir, "config.json"), encoding="utf-8") as fh:
        return json.load(fh)["architectures"]


# ------------------------------------------------------------------------------------------- conversion
def recover_original_state_dict_from_checkpoint(sd: Dict[str, torch.Tensor], pretrained_model_name_or_path: str = None,
                                                weight_map: Optional[Dict[str, str]] = None,
                                                architectures: Optional[List[str]] = None) -> Dict[str, torch.Tensor]:
    """Rewrite every ScatterMoE block of ``sd`` into the parameter names / layouts of the original checkpoint."""
    if weight_map is None:
        weight_map = load_weight_map(get_resolved_checkpoint_location(pretrained_model_name_or_path))
    if architectures is None:
        architectures = _read_architectures(pretrained_model_name_or_path)
    _, router_name, expert_name, _, sharded_experts = get_scattermoe_conv_spec_from_archs(architectures)

    names = "|".join([PARAM_NAME_ROUTER_SCATTERMOE, *PARAM_NAME_WEIGHT_SCATTERMOE])
    pat = re.compile(rf"(.*)\.({names})\.weight")
    seen: Dict[str, int] = defaultdict(int)
    for k in sd:
        m = pat.match(k)
        if m:
            seen[m.group(1)] += 1
    for full_prefix in [p for p, c in seen.items() if c >= 3]:
        prefix, _, module_name = full_prefix.rpartition(".")
        meta = get_checkpoint_meta_from_sharded_safetensor(weight_map, prefix, module_name, router_name, expert_name)
        per_model_key: Dict[str, Dict[str, torch.Tensor]] = defaultdict(dict)
        for scatter_key, targets in meta.items():
            fq = f"{full_prefix}.{scatter_key}"
            param = sd.pop(fq)
            n = len(targets)
            is_expert = any(scatter_key.startswith(w) for w in PARAM_NAME_WEIGHT_SCATTERMOE)
            if not is_expert:
                assert n == 1, "Router parameters should not be sharded."
            elif not sharded_experts:
                assert n == 1, "Expert weights expected to be non-sharded."
            else:
                # one tensor per expert, or (transformers >= 5 layout of the same family) one fused 3-D tensor
                assert n in (1, param.shape[0]), "Sharded expert weights should be 1 expert per shard."
            if is_expert:
                param = param.permute(0, 2, 1)  # [E, in, out] -> [E, out, in]
            for i, (model_key, _) in enumerate(targets):
                per_model_key[model_key][scatter_key] = param if n == 1 else param[i]
        for model_key, parts in per_model_key.items():
            keys = sorted(parts)  # w1 before w3: the fused input projection is [w1 rows | w3 rows]
            assert keys, f"Obtained zero scatter keys for model_key '{model_key}'"
            sd[model_key] = parts[keys[0]].contiguous() if len(keys) == 1 else torch.cat([parts[k] for k in keys], dim=1)
    return sd


def save_sharded_safetensors(input_state_dict: Dict[str, torch.Tensor], save_directory: str,
                             metadata: Optional[Dict] = None, max_shard_size="5GB", lora: bool = False) -> None:
    from safetensors.torch import save_file

    from ...peft.gptqmodel.utils.model import parse_size, shard_checkpoint

    os.makedirs(save_directory, exist_ok=True)
    sd = {k: v.detach().cpu().contiguous() for k, v in input_state_dict.items()}
    meta = dict(metadata or {"format": "pt"})
    if lora:
        save_file(sd, os.path.join(save_directory, ADAPTER_SAFE_WEIGHTS_NAME), metadata=meta)
        return
    shards, index = shard_checkpoint(sd, parse_size(max_shard_size), SAFE_WEIGHTS_NAME)
    for fname, part in shards.items():
        save_file(part, os.path.join(save_directory, fname), metadata=meta)
    if index is not None:
        with open(os.path.join(save_directory, FILE_SAFETENSOR_INDEX), "w", encoding="utf-8") as fh:
            json.dump(index, fh, indent=2, sort_keys=True)


def recover_safetensors_from_dcp(checkpoint_dir: str, pretrained_model_name_or_path: Optional[str], output_dir: str) -> None:
    """DCP (or safetensors) training checkpoint -> Hugging Face safetensors in the original parameter layout."""
    fsdp_dirs = sorted(d for d in os.listdir(checkpoint_dir) if d.startswith(FSDP_MODEL_NAME))
    if len(fsdp_dirs) > 1:
        raise ValueError(f"Found > 1 dirs in dcp checkpoint dir {checkpoint_dir}: {fsdp_dirs}. Please spectify the exact one.")
    if fsdp_dirs:
        sd = get_state_dict_from_dcp_checkpoint(os.path.join(checkpoint_dir, fsdp_dirs[0]))
    else:
        sd = get_state_dict_from_safe_checkpoint(checkpoint_dir)
    # strip PEFT naming: "base_model.model." prefix and the ".default" adapter infix
    lora = False
    cleaned = {}
    for k, v in sd.items():
        if "lora_A" in k or "lora_B" in k:
            lora = True
        nk = k[len("base_model.model."):] if (k.startswith("base_model.model.") and not ("lora_" in k)) else k
        nk = nk.replace(".default.", ".").replace(".base_layer.", ".")
        cleaned[nk] = v
    sd = cleaned
    if pretrained_model_name_or_path is not None and not lora:
        if os.path.isdir(pretrained_model_name_or_path):
            sd = recover_original_state_dict_from_checkpoint(sd, pretrained_model_name_or_path)
        else:
            # a run that started from an architecture preset (random-init weights): the original parameter names
            # and the architecture come from the preset's model skeleton instead of from checkpoint files
            from ....models.builder import build_model, resolve_config

            cfg = resolve_config(pretrained_model_name_or_path)
            with torch.device("meta"):
                skeleton = build_model(cfg, device="meta", dtype=torch.bfloat16)
            sd = recover_original_state_dict_from_checkpoint(
                sd, weight_map={k: SAFE_WEIGHTS_NAME for k in skeleton.state_dict()}, architectures=list(cfg.architectures))
    save_sharded_safetensors({k: v.contiguous() for k, v in sd.items()}, output_dir, metadata={"format": "pt"}, lora=lora)


def main(argv=None) -> int:
    import argparse

    ap = argparse.ArgumentParser(description="Convert a ScatterMoE training checkpoint to Hugging Face safetensors")
    ap.add_argument("checkpoint_dir", help="directory that holds pytorch_model_fsdp_<i>/ (or safetensors files)")
    ap.add_argument("output_dir")
    ap.add_argument("pretrained_model_name_or_path", nargs="?", default=None,
                    help="original checkpoint (for the parameter names and layout); optional for LoRA checkpoints")
    a = ap.parse_args(argv)
    recover_safetensors_from_dcp(a.checkpoint_dir, a.pretrained_model_name_or_path, a.output_dir)
    return 0


if __name__ == "__main__":
    sys.exit(main())
