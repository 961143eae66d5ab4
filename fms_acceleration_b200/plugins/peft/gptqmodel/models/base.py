"""``BaseGPTQModel``: quantise a float model layer by layer, save it in the GPTQ checkpoint layout, load it back.

Checkpoint contract (fms_acceleration_peft/gptqmodel/models/base.py:548-769 of the reference): weights in
``model.safetensors`` (or shards + ``model.safetensors.index.json``) with metadata ``{"format": "pt"}``, the
quantisation description both in ``quantize_config.json`` and in ``config.json["quantization_config"]``.
Loading (``:775-1300``): build the float skeleton, swap the per-family linears for ``QuantLinear``, load the
tensors, and account for the v1 zero-point layout (``zero - 1``) of older checkpoints.
"""
from __future__ import annotations

import copy
import json
import os
from typing import Dict, List, Optional, Union

import torch
from torch import nn

from fms_acceleration_b200.models.builder import build_model, resolve_config
from fms_acceleration_b200.nn.gptq import QuantLinear
from ..quantization.config import FORMAT, META_FIELD_QUANTIZER, META_QUANTIZER_NAME, QuantizeConfig
from ..quantization.gptq import GPTQ
from ..utils.backend import Backend
from ..utils.data import collate_data
from ..utils.model import (SAFE_WEIGHTS_INDEX_NAME, SAFE_WEIGHTS_NAME, convert_gptq_v1_to_v2_format, find_layers,
                           get_checkpoints, make_quant, pack_model, parse_size, recurse_getattr, shard_checkpoint)


class _StopForward(Exception):
    pass


class BaseGPTQModel(nn.Module):
    base_modules: List[str] = None
    lm_head: str = "lm_head"
    layers_node: str = None
    layer_type: str = None
    layer_modules: List[List[str]] = None
    dynamic_expert_index: Optional[str] = None
    info: Dict[str, str] = {}
    # families whose Hugging Face implementation is remote code ask for ``trust_remote_code=True`` when loading
    require_trust_remote_code = None

    def __init__(self, model: nn.Module, quantized: bool, quantize_config: QuantizeConfig):
        super().__init__()
        self.model = model
        self._quantized = quantized
        self.quantize_config = quantize_config
        self.config = getattr(model, "config", None)

    @property
    def quantized(self) -> bool:
        return self._quantized

    def forward(self, *args, **kwargs):
        return self.model(*args, **kwargs)

    def to(self, device):
        self.model.to(device)
        return self

    @property
    def hf_device_map(self):
        return getattr(self.model, "hf_device_map", None)

    @property
    def device(self) -> torch.device:
        placement = self.hf_device_map
        if placement:
            return torch.device(next(d for d in placement.values() if d != "disk"))
        inner = getattr(self.model, "device", None)
        return inner if isinstance(inner, torch.device) else next(self.model.parameters()).device

    def generate(self, **kwargs):
        """Shortcut for ``model.generate`` under inference mode and autocast."""
        with torch.inference_mode(), torch.amp.autocast(device_type=self.device.type):
            return self.model.generate(**kwargs)

    def prepare_inputs_for_generation(self, *args, **kwargs):
        return self.model.prepare_inputs_for_generation(*args, **kwargs)

    def shard_checkpoint(self, state_dict: Dict[str, torch.Tensor], max_shard_size: Union[int, str] = "10GB",
                         weights_name: str = SAFE_WEIGHTS_NAME):
        """``(shards: file name -> tensors, index or None)``: tensors in key order, a new file whenever the next
        tensor would take the current one over ``max_shard_size`` (a larger single tensor gets a file of its own)."""
        return shard_checkpoint(state_dict, parse_size(max_shard_size), weights_name)

    def warmup_triton(self, enabled: bool = True):
        """Kept for call compatibility: the CUDA kernels here have no autotuning cache to fill."""
        if enabled:
            QuantLinear.warmup(self.model, seqlen=getattr(self.model, "seqlen", 2048))

    def __getattr__(self, item):
        try:
            return super().__getattr__(item)
        except AttributeError:
            if item == "model":
                raise
            return getattr(self.model, item)

    # ------------------------------------------------------------------ helpers
    @classmethod
    def expanded_layer_modules(cls, config) -> List[List[str]]:
        """Per-layer module groups with ``{expert_index}`` expanded for MoE families."""
        if cls.dynamic_expert_index is None:
            return cls.layer_modules
        n = config
        for part in cls.dynamic_expert_index.split("."):
            n = getattr(n, part)
        out = []
        for group in cls.layer_modules:
            g = []
            for name in group:
                if "{expert_index}" in name:
                    g += [name.format(expert_index=i) for i in range(int(n))]
                else:
                    g.append(name)
            out.append(g)
        return out

    def _quant_targets(self, model) -> List[str]:
        layers = recurse_getattr(model, self.layers_node)
        names = []
        groups = self.expanded_layer_modules(model.config)
        for i in range(len(layers)):
            for g in groups:
                names += [f"{self.layers_node}.{i}.{n}" for n in g]
        if self.quantize_config.lm_head:
            names.append(self.lm_head)
        return names

    # ------------------------------------------------------------------ quantise
    @torch.no_grad()
    def quantize(self, calibration_dataset: List[Dict[str, Union[List[int], torch.Tensor]]], batch_size: int = 1,
                 calibration_enable_gpu_cache: bool = True):
        if self.quantized:
            raise EnvironmentError("quantize() is called a model that is already quantized")
        if not calibration_dataset:
            raise ValueError("Calibration dataset must not be empty.")
        qc = self.quantize_config
        model = self.model
        model.eval()
        layers = recurse_getattr(model, self.layers_node)
        dev = next(model.parameters()).device
        batches = [collate_data(calibration_dataset[i: i + batch_size], 0)
                   for i in range(0, len(calibration_dataset), batch_size)]

        # capture the inputs of the first decoder layer
        captured = []

        def grab(mod, args, kwargs):
            captured.append((tuple(a.detach() if torch.is_tensor(a) else a for a in args),
                             {k: (v.detach() if torch.is_tensor(v) else v) for k, v in kwargs.items()}))
            raise _StopForward

        handle = layers[0].register_forward_pre_hook(grab, with_kwargs=True)
        for b in batches:
            try:
                model(b["input_ids"].to(dev))
            except _StopForward:
                pass
        handle.remove()

        quantizers = {}
        groups = self.expanded_layer_modules(model.config)
        layer_inputs = captured
        for li, layer in enumerate(layers):
            full = find_layers(layer)
            for names in groups:
                subset = {n: full[n] for n in names if n in full}
                if not subset:
                    continue
                gptq = {}
                for n, lin in subset.items():
                    g = GPTQ(lin)
                    g.quantizer.configure(qc.bits, perchannel=True, sym=qc.sym, mse=False)
                    gptq[n] = g
                hooks = [lin.register_forward_hook(
                    (lambda name: (lambda m, inp, out: gptq[name].add_batch(inp[0].data, out.data)))(n))
                    for n, lin in subset.items()]
                for args, kwargs in layer_inputs:
                    layer(*args, **kwargs)
                for h in hooks:
                    h.remove()
                for n in subset:
                    scale, zero, g_idx, _, _ = gptq[n].fasterquant(
                        percdamp=qc.damp_percent, group_size=qc.group_size, actorder=qc.desc_act,
                        static_groups=qc.static_groups)
                    quantizers[f"{self.layers_node}.{li}.{n}"] = (gptq[n].quantizer, scale.cpu(), zero.cpu(), g_idx.cpu())
                    gptq[n].free()
            # outputs of this (now quantised) layer feed the next one
            nxt = []
            for args, kwargs in layer_inputs:
                out = layer(*args, **kwargs)
                out = out[0] if isinstance(out, tuple) else out
                nxt.append(((out,) + tuple(args[1:]), kwargs))
            layer_inputs = nxt

        dtype = next(model.parameters()).dtype
        pack_model(model, quantizers, qc.bits, qc.group_size, dtype if dtype in (torch.float16, torch.bfloat16) else torch.float16)
        self._quantized = True
        qc.format = FORMAT.GPTQ_V2
        return quantizers

    # ------------------------------------------------------------------ save
    def save_quantized(self, save_dir: str, safetensors_metadata: Optional[Dict[str, str]] = None,
                       use_safetensors: bool = True, max_shard_size: Optional[Union[int, str]] = None,
                       model_base_name: Optional[str] = None):
        from safetensors.torch import save_file

        if not self.quantized:
            raise EnvironmentError("can only save quantized model, please execute .quantize first.")
        os.makedirs(save_dir, exist_ok=True)
        qc = copy.deepcopy(self.quantize_config)
        qc.meta_set_versionable(META_FIELD_QUANTIZER, META_QUANTIZER_NAME, "0.1.0")
        state = {}
        seen = {}
        for k, v in self.model.state_dict().items():
            key = (v.data_ptr(), v.numel())
            if v.numel() and key in seen:
                continue  # tied weights are stored once
            seen[key] = k
            state[k] = v.detach().cpu().contiguous()
        name = (model_base_name + ".safetensors") if model_base_name else SAFE_WEIGHTS_NAME
        meta = {"format": "pt"}
        meta.update({str(k): str(v) for k, v in (safetensors_metadata or {}).items()})
        limit = parse_size(max_shard_size) if max_shard_size is not None else 2 ** 62
        shards, index = shard_checkpoint(state, limit, name)
        for fname, sd in shards.items():
            save_file(sd, os.path.join(save_dir, fname), metadata=meta)
        if index is not None:
            with open(os.path.join(save_dir, SAFE_WEIGHTS_INDEX_NAME), "w", encoding="utf-8") as fh:
                json.dump(index, fh, indent=2)
        cfg = self.model.config.to_dict() if hasattr(self.model.config, "to_dict") else dict(vars(self.model.config))
        cfg["quantization_config"] = qc.to_dict()
        with open(os.path.join(save_dir, "config.json"), "w", encoding="utf-8") as fh:
            json.dump(cfg, fh, indent=2)
        qc.model_name_or_path = save_dir
        qc.model_file_base_name = os.path.splitext(name)[0]
        qc.save_pretrained(save_dir)

    def save_pretrained(self, save_dir: str, **kwargs):
        self.save_quantized(save_dir, **kwargs)

    # ------------------------------------------------------------------ load
    @classmethod
    def from_pretrained(cls, pretrained_model_name_or_path, quantize_config: QuantizeConfig,
                        torch_dtype=torch.float32, device="cpu", **kwargs):
        cls._check_remote_code(pretrained_model_name_or_path, kwargs.get("trust_remote_code", False))
        model = build_model(pretrained_model_name_or_path, device=device, dtype=torch_dtype)
        return cls(model, False, quantize_config)

    @classmethod
    def _check_remote_code(cls, name, trust_remote_code: bool) -> None:
        if cls.require_trust_remote_code and not trust_remote_code:
            raise ValueError(f"{name} requires trust_remote_code=True. Please set trust_remote_code=True to load this model.")

    @classmethod
    def from_quantized(cls, model_name_or_path, quantize_config: Optional[QuantizeConfig] = None,
                       backend: Backend = Backend.AUTO, torch_dtype=torch.float16, device=None,
                       low_cpu_mem_usage: bool = False, **kwargs):
        from safetensors.torch import load_file

        cls._check_remote_code(model_name_or_path, kwargs.get("trust_remote_code", False))
        device = device if device is not None else "cpu"
        cfg = resolve_config(model_name_or_path)
        is_dir = isinstance(model_name_or_path, str) and os.path.isdir(model_name_or_path)
        if quantize_config is None:
            if not is_dir:
                raise ValueError("quantize_config is required when the model is not a checkpoint directory")
            quantize_config = QuantizeConfig.from_pretrained(model_name_or_path)
        qc = quantize_config
        v1_layout = qc.format in (FORMAT.GPTQ, FORMAT.TRITON) and not qc.is_quantized_or_packed_by_v2()
        files: List[str] = []
        if is_dir:
            _, files, _ = get_checkpoints(model_name_or_path)
        zero_offset = 1 if (v1_layout and files) else 0
        groups = cls.expanded_layer_modules(cfg)
        gen = torch.Generator(device=device) if not files else None
        if gen is not None:
            gen.manual_seed(int(kwargs.get("seed", 0)))

        def to_quant(layer):
            for g in groups:
                for n in g:
                    try:
                        lin = recurse_getattr(layer, n)
                    except AttributeError:
                        continue
                    if files:
                        make_quant(layer, [n], qc.bits, qc.group_size, torch_dtype, zero_offset, device)
                    else:
                        # no weights on disk: random codes / scales as the synthetic benchmark configuration defines
                        from ..utils.model import recurse_setattr

                        recurse_setattr(layer, n, QuantLinear.random(lin.in_features, lin.out_features, qc.bits,
                                                                     qc.group_size, torch_dtype, device, gen))
            return layer

        model = build_model(cfg, device=device, dtype=torch_dtype, layer_hook=to_quant)
        if files:
            state = {}
            for f in files:
                state.update(load_file(f, device=str(device)))
            missing, unexpected = model.load_state_dict(state, strict=False)
            missing = [m for m in missing if not (m.endswith("lm_head.weight") and cfg.tie_word_embeddings)]
            if missing:
                raise ValueError(f"checkpoint is missing tensors: {missing[:8]}{'...' if len(missing) > 8 else ''}")
            for m in model.modules():
                if isinstance(m, QuantLinear):
                    m.post_init()
            if zero_offset:
                convert_gptq_v1_to_v2_format(model, qc.bits)
        return cls(model, True, qc)
