"""Model surgery helpers for GPTQ: locate linears, swap them for ``QuantLinear``, pack, convert between the
v1 and v2 zero-point layouts, find and shard checkpoint files.  Role of
fms_acceleration_peft/gptqmodel/utils/model.py:103-717 in the reference."""
from __future__ import annotations

import json
import os
import re
from typing import Dict, List, Optional, Tuple

import torch
from torch import nn

from fms_acceleration_b200.nn.gptq import QuantLinear

SAFE_WEIGHTS_NAME = "model.safetensors"
SAFE_WEIGHTS_INDEX_NAME = "model.safetensors.index.json"


def recurse_getattr(obj, attr: str):
    for part in attr.split("."):
        obj = getattr(obj, part)
    return obj


def recurse_setattr(module, name: str, value) -> None:
    head, _, leaf = name.rpartition(".")
    target = recurse_getattr(module, head) if head else module
    setattr(target, leaf, value)


def find_layers(module: nn.Module, layers=None, name: str = "") -> Dict[str, nn.Module]:
    """All (dotted name -> module) below ``module`` whose type is one of ``layers`` (default: linear-like)."""
    if layers is None:
        layers = (nn.Linear, nn.Conv2d)
    found = {}
    for n, m in module.named_modules():
        if isinstance(m, tuple(layers)) or (m.__class__.__name__ == "Conv1D" and nn.Linear in layers):
            found[(name + "." + n) if name and n else (n or name)] = m
    return found


def get_module_by_name_prefix(model: nn.Module, prefix: str):
    for n, m in model.named_modules():
        if n.startswith(prefix):
            return m
    return None


def get_module_by_name_suffix(model: nn.Module, suffix: str):
    for n, m in model.named_modules():
        if n.endswith(suffix):
            return m
    return None


def make_quant(module: nn.Module, names, bits: int, group_size: int, dtype=torch.float16, zero_offset: int = 0,
               device=None) -> None:
    """Replace the linears listed in ``names`` (dotted, relative to ``module``) by empty ``QuantLinear``s."""
    for n in list(names):
        sub = recurse_getattr(module, n)
        if isinstance(sub, QuantLinear):
            continue
        if isinstance(sub, nn.Linear):
            in_f, out_f = sub.in_features, sub.out_features
        elif sub.__class__.__name__ == "Conv1D":
            in_f, out_f = sub.weight.shape[0], sub.weight.shape[1]
        else:
            in_f, out_f = sub.in_channels, sub.out_channels
        dev = device if device is not None else (sub.weight.device if not sub.weight.is_meta else "cpu")
        ql = QuantLinear(bits, group_size, in_f, out_f, getattr(sub, "bias", None) is not None, dtype, zero_offset, dev)
        recurse_setattr(module, n, ql)


def pack_model(model: nn.Module, quantizers: Dict[str, Tuple], bits: int, group_size: int, dtype=torch.float16) -> None:
    """``quantizers[name] = (quantizer, scale [out,G], zero [out,G], g_idx)`` -> packed ``QuantLinear`` modules."""
    floats = {n: m for n, m in find_layers(model).items() if n in quantizers}
    make_quant(model, floats.keys(), bits, group_size, dtype)
    for name, lin in floats.items():
        _, scale, zero, g_idx = quantizers[name]
        ql: QuantLinear = recurse_getattr(model, name)
        ql.pack(lin.to("cpu"), scale.to("cpu"), zero.to("cpu"), g_idx.to("cpu") if g_idx is not None else None)


def convert_gptq_v1_to_v2_format(model: nn.Module, bits: int) -> nn.Module:
    """v1 checkpoints store ``zero - 1``; add one to every packed zero field (an integer add of a repeated
    ``1`` pattern, e.g. 0x11111111 for 4 bits, carries exactly like the reference's conversion)."""
    pattern = {2: 0b01010101010101010101010101010101, 4: 0x11111111, 8: 0x01010101}
    for m in model.modules():
        if isinstance(m, QuantLinear):
            if bits == 3:
                raise NotImplementedError("3-bit zero-point conversion is not supported")
            add = pattern[bits]
            z = (m.qzeros.long() & 0xFFFFFFFF) + add
            z = z & 0xFFFFFFFF
            m.qzeros = torch.where(z >= 2 ** 31, z - 2 ** 32, z).to(torch.int32)
            m.zero_offset = 0
    return model


def convert_gptq_v2_to_v1_format(model: nn.Module, bits: int) -> nn.Module:
    pattern = {2: 0b01010101010101010101010101010101, 4: 0x11111111, 8: 0x01010101}
    for m in model.modules():
        if isinstance(m, QuantLinear):
            sub = pattern[bits]
            z = ((m.qzeros.long() & 0xFFFFFFFF) - sub) & 0xFFFFFFFF
            m.qzeros = torch.where(z >= 2 ** 31, z - 2 ** 32, z).to(torch.int32)
            m.zero_offset = 1
    return model


def get_checkpoints(model_dir: str, extensions=(".safetensors",), possible_basenames=("model", "gptq_model"),
                    **kwargs) -> Tuple[bool, List[str], Optional[str]]:
    """(is_sharded, files, found_basename) for a local checkpoint directory."""
    index = os.path.join(model_dir, SAFE_WEIGHTS_INDEX_NAME)
    if os.path.exists(index):
        with open(index, encoding="utf-8") as fh:
            files = sorted(set(json.load(fh)["weight_map"].values()))
        return True, [os.path.join(model_dir, f) for f in files], "model"
    for base in possible_basenames:
        for ext in extensions:
            p = os.path.join(model_dir, base + ext)
            if os.path.exists(p):
                return False, [p], base
    return False, [], None


def shard_checkpoint(state_dict: Dict[str, torch.Tensor], max_shard_size: int = 5 * 2 ** 30,
                     weights_name: str = SAFE_WEIGHTS_NAME):
    """Split a state dict into shards of at most ``max_shard_size`` bytes.  Returns (shards, index or None)."""
    shards: List[Dict[str, torch.Tensor]] = [{}]
    sizes = [0]
    total = 0
    for k, v in state_dict.items():
        nbytes = v.numel() * v.element_size()
        if sizes[-1] + nbytes > max_shard_size and shards[-1]:
            shards.append({})
            sizes.append(0)
        shards[-1][k] = v
        sizes[-1] += nbytes
        total += nbytes
    if len(shards) == 1:
        return {weights_name: shards[0]}, None
    stem, ext = os.path.splitext(weights_name)
    named, weight_map = {}, {}
    for i, sh in enumerate(shards):
        fname = f"{stem}-{i + 1:05d}-of-{len(shards):05d}{ext}"
        named[fname] = sh
        for k in sh:
            weight_map[k] = fname
    return named, {"metadata": {"total_size": total}, "weight_map": weight_map}


def parse_size(size) -> int:
    if isinstance(size, int):
        return size
    m = re.fullmatch(r"\s*(\d+(?:\.\d+)?)\s*([KMGT]?)I?B\s*", str(size).upper())
    if not m:
        raise ValueError(f"cannot parse size {size!r}")
    mult = {"": 1, "K": 2 ** 10, "M": 2 ** 20, "G": 2 ** 30, "T": 2 ** 40}[m.group(2)]
    return int(float(m.group(1)) * mult)


def auto_dtype_from_config(config, quant_inference: bool = False) -> torch.dtype:
    dt = getattr(config, "torch_dtype", None)
    if isinstance(dt, str):
        dt = getattr(torch, dt, None)
    if dt in (torch.float16, torch.bfloat16):
        return dt
    return torch.float16


EXPERT_INDEX_PLACEHOLDER = "{expert_index}"


def get_moe_layer_modules(layer_modules: List[List[str]], num_experts: int) -> List[List[str]]:
    """Expand every name that carries ``{expert_index}`` into one name per expert, keeping the grouping of the
    per-layer quantisation order (fms_acceleration_peft/gptqmodel/utils/model.py:704-717)."""
    out: List[List[str]] = []
    for group in layer_modules:
        expanded: List[str] = []
        for name in group:
            if EXPERT_INDEX_PLACEHOLDER in name:
                expanded += [name.replace(EXPERT_INDEX_PLACEHOLDER, str(e)) for e in range(num_experts)]
            else:
                expanded.append(name)
        out.append(expanded)
    return out


def simple_dispatch_model(model: nn.Module, device_map: Dict[str, str]) -> nn.Module:
    """Place a model according to a device map (fms_acceleration_peft/gptqmodel/utils/model.py:407-448).

    One GPU holds a whole 70B GPTQ model here, so only two kinds of map are meaningful: ``{"": device}`` moves
    everything, and a per-module map moves each named sub-tree to its device and makes the module's forward
    bring its inputs along.  Offload to "cpu"/"disk" with execution elsewhere is not provided."""
    if "" in device_map:
        model = model.to(torch.device(device_map[""]))
        model.hf_device_map = dict(device_map)
        return model
    if any(d in ("cpu", "disk") for d in device_map.values()) and len(set(device_map.values())) > 1:
        raise NotImplementedError("offloaded execution is not provided; map every module to one accelerator")
    tied = find_tied_parameters(model)
    for name, dev in device_map.items():
        mod = get_module_by_name_suffix(model, name)
        if mod is None:
            raise KeyError(f"device_map names {name!r}, which the model does not have")
        target = torch.device(dev)
        mod.to(target)

        def _pre(_m, args, kwargs, _t=target):
            mv = lambda v: v.to(_t) if isinstance(v, torch.Tensor) else v  # noqa: E731
            return tuple(mv(a) for a in args), {k: mv(v) for k, v in kwargs.items()}

        mod.register_forward_pre_hook(_pre, with_kwargs=True)
    retie_parameters(model, tied)
    model.hf_device_map = dict(device_map)
    return model


def find_tied_parameters(model: nn.Module) -> List[List[str]]:
    """Groups of parameter names that share one storage."""
    seen: Dict[int, List[str]] = {}
    for name, p in model.named_parameters(remove_duplicate=False):
        seen.setdefault(id(p), []).append(name)
    return [names for names in seen.values() if len(names) > 1]


def retie_parameters(model: nn.Module, tied: List[List[str]]) -> None:
    for names in tied:
        src = recurse_getattr(model, names[0])
        for other in names[1:]:
            recurse_setattr(model, other, src)


def verify_file_hash(path: str, expected: str) -> bool:
    """``expected`` is ``"<algorithm>:<hex digest>"`` (md5, sha256 ...); the file is read in 1 MiB pieces."""
    import hashlib

    algo, _, digest = expected.partition(":")
    if not digest or algo.lower() not in hashlib.algorithms_available:
        raise ValueError(f"hash must look like 'sha256:<hex>', got {expected!r}")
    h = hashlib.new(algo.lower())
    with open(path, "rb") as fh:
        for piece in iter(lambda: fh.read(1 << 20), b""):
            h.update(piece)
    return h.hexdigest() == digest.lower()


# ------------------------------------------------------------------------------------------------
# Small helpers with the reference's names (fms_acceleration_peft/gptqmodel/utils/model.py:82-100, 272-290, 367-404,
# 455-520), so that code written against its GPTQ library keeps importing.
# ------------------------------------------------------------------------------------------------
def get_device(obj) -> torch.device:
    """Device of a tensor, or of a module's first parameter (buffers when it has no parameter)."""
    if isinstance(obj, torch.Tensor):
        return obj.device
    for t in obj.parameters():
        return t.device
    for t in obj.buffers():
        return t.device
    raise ValueError("the module holds no tensor")


def move_to(obj, device):
    """``obj`` on ``device``; tensors and modules already there are returned as they are."""
    device = torch.device(device)
    return obj if get_device(obj) == device else obj.to(device)


def nested_move_to(value, device):
    """:func:`move_to` through lists, tuples and dicts; anything that is not a tensor is passed through."""
    if isinstance(value, torch.Tensor):
        return move_to(value, device)
    if isinstance(value, (list, tuple)):
        return type(value)(nested_move_to(v, device) for v in value)
    if isinstance(value, dict):
        return {k: nested_move_to(v, device) for k, v in value.items()}
    return value


def select_quant_linear_with_pack(bits: int, group_size: int, desc_act: bool, sym: bool, backend=None,
                                  format: str = None, pack: bool = True):
    """The ``QuantLinear`` class for these settings that can also pack a float layer."""
    from ..quantization.config import FORMAT
    from .backend import Backend
    from .importer import select_quant_linear

    return select_quant_linear(bits=bits, group_size=group_size, desc_act=desc_act, sym=sym,
                               backend=backend if backend is not None else Backend.AUTO,
                               format=format if format is not None else FORMAT.GPTQ_V2, pack=pack)


def verify_model_hash(file_path: str, verify_hash: str) -> bool:
    """``verify_hash`` is ``"<algorithm>:<hex digest>"``."""
    if not isinstance(verify_hash, str):
        raise ValueError("model verify_hash must be a string")
    if ":" not in verify_hash:
        raise ValueError("verify_hash must be in the format 'hash_type:hash_value'")
    return verify_file_hash(file_path, verify_hash)


def verify_sharded_model_hashes(index_json: str, verify_hash: List[str]) -> bool:
    """One hash per shard file named in a ``*.index.json`` weight map (shards in sorted order, resolved beside the
    index file)."""
    if not isinstance(verify_hash, list):
        raise ValueError("sharded model verify_hash must be a list")
    with open(index_json, encoding="utf-8") as fh:
        shards = sorted(set(json.load(fh)["weight_map"].values()))
    if len(shards) != len(verify_hash):
        raise ValueError("Number of shards and number of hash values do not match.")
    folder = os.path.dirname(os.path.abspath(index_json))
    return all(verify_model_hash(os.path.join(folder, shard), h) for shard, h in zip(shards, verify_hash))


def check_and_get_model_type(model_dir: str, trust_remote_code: bool = False) -> str:
    """``model_type`` of the configuration in ``model_dir`` if the GPTQ library has a class for it."""
    from ..models.auto import MODEL_MAP

    with open(os.path.join(model_dir, "config.json"), encoding="utf-8") as fh:
        model_type = json.load(fh).get("model_type")
    if model_type not in MODEL_MAP:
        raise TypeError(f"{model_type} isn't supported yet.")
    return model_type


def gptqmodel_post_init(model: nn.Module, use_act_order: bool = False, max_input_length: Optional[int] = None) -> nn.Module:
    """Run ``post_init`` of every quantised linear (here: decide whether its groups are in input order, which selects
    the kernels).  The reference's scratch buffers for the exllama kernels have no counterpart."""
    for m in model.modules():
        if isinstance(m, QuantLinear):
            m.post_init()
    return model
