"""Library-kernel execution of the in-tree decoder models (the same-box comparison arm).

What runs where:

* projections: ``torch.matmul`` (cuBLAS).  A frozen 4-bit weight is expanded to 16 bits before every use, in forward
  and again in backward, which is what bitsandbytes' ``matmul_4bit`` does for the reference.  bitsandbytes itself
  is not installable here, so the expansion uses this package's dequantise kernel; the LoRA update is plain torch
  ops on the side (``x A^T B^T`` times the scale), as in peft.
* attention: ``flash_attn_varlen_func`` of the installed flash-attn (what the reference's padding-free plugin
  calls, fms_acceleration_aadp/flash_attn.py), rotary embedding with explicit position ids in torch ops (the
  reference's Triton RoPE assumes ``position = row % seqlen`` and is therefore not usable on packed batches).
* RMSNorm, SwiGLU, fused linear + cross-entropy: the reference's OWN Triton kernels, loaded by file path from an
  unmodified copy of the reference under ``baseline/_ref`` (``fms_acceleration_foak/kernels/unsloth/
  rms_layernorm.py``, ``fused_ops/unsloth_lora/swiglu.py``, ``fused_ops/liger_ce/fused_linear_cross_entropy_loss.py``).
  Where a file cannot be loaded (no copy, or no GPU), the torch formulation of the same operation is used and
  :func:`reference_kernels_status` says so.
* mixture-of-experts blocks: the reference's ScatterMoE Triton kernels (``scattered_experts`` of
  ``fms_acceleration_moe/utils/scattermoe_utils/khd/kernels/ops``, loaded by path) wired as the reference's
  ``ScatterMoE.forward`` wires them (scattermoe.py:411-491): sort the (token, expert) pairs, padded block indices,
  scatter-to-scatter up / gate projections, grouped down projection with the routing weights.  Under expert
  parallelism the rows are exchanged with ``all_to_all_single`` over NCCL first (the exchange of the reference's
  scattermoe_utils/expert_parallel.py) and the kernels run on the received rows, already grouped by expert.  If the
  files cannot be loaded: per-expert ``torch.matmul`` (the ``ScatterMoE`` module's ``library`` backend).
* gradient synchronisation: the engine's ``library`` backend (NCCL all-reduce).

Parameters are shared with the model the runner is built from; nothing is copied.
"""
from __future__ import annotations

import importlib
import os
import sys
import types
from typing import Dict, Optional

import torch
import torch.nn.functional as F
from torch import nn

REPO = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
REF_ROOT = os.path.join(REPO, "baseline", "_ref")
IGNORE = -100

_STATUS: Dict[str, str] = {}
_MODS: Dict[str, object] = {}


def _load_reference(package: str, dotted: str):
    """Import ``<package>.<dotted>`` from the reference copy WITHOUT running the ``__init__`` files of the packages
    on the way (they import peft / accelerate / bitsandbytes): every package level is registered as an empty module
    that only knows its directory, then the leaf file is imported normally, so its relative imports resolve."""
    key = f"{package}.{dotted}"
    if key in _MODS:
        return _MODS[key]
    root_dir = os.path.join(REF_ROOT, package)
    if not os.path.isdir(root_dir):
        raise FileNotFoundError(f"no copy of the reference package {package!r} under baseline/_ref")
    alias = "fmsb_ref_" + package
    parts = dotted.split(".")
    name, path = alias, root_dir
    for i in range(len(parts)):
        if name not in sys.modules:
            mod = types.ModuleType(name)
            mod.__path__ = [path]
            mod.__package__ = name
            sys.modules[name] = mod
        if i < len(parts) - 1:
            name, path = f"{name}.{parts[i]}", os.path.join(path, parts[i])
    mod = importlib.import_module(f"{alias}.{dotted}")
    _MODS[key] = mod
    return mod


def _try(tag: str, package: str, dotted: str):
    try:
        mod = _load_reference(package, dotted)
        _STATUS[tag] = "reference Triton kernel (loaded by path)"
        return mod
    except Exception as exc:  # no copy, no triton, no GPU...
        _STATUS[tag] = f"torch formulation ({type(exc).__name__}: {str(exc)[:120]})"
        return None


def reference_kernels_status() -> Dict[str, str]:
    """Which of the reference's kernel files the baseline is actually running."""
    return dict(_STATUS)


# ------------------------------------------------------------------------------------------------ building blocks
class _FrozenMatmul(torch.autograd.Function):
    """y = x W^T for a frozen quantised module: W is expanded on the fly in forward and again in backward."""

    @staticmethod
    def forward(ctx, x, mod):
        ctx.mod = mod
        return x @ mod.dequantize(dtype=x.dtype).t()

    @staticmethod
    def backward(ctx, dy):
        return dy @ ctx.mod.dequantize(dtype=dy.dtype), None


def _linear(mod: nn.Module, x: torch.Tensor) -> torch.Tensor:
    if hasattr(mod, "base_layer") and hasattr(mod, "lora_A"):  # LoRA wrapper: base + scale * B(A(x))
        y = _linear(mod.base_layer, x)
        for name, A in mod.lora_A.items():
            B = mod.lora_B[name]
            y = y + ((x @ A.weight.t()) @ B.weight.t()) * mod.scaling[name]
        return y
    if hasattr(mod, "dequantize"):
        y = _FrozenMatmul.apply(x, mod)
    else:
        y = x @ mod.weight.t()
    b = getattr(mod, "bias", None)
    return y if b is None else y + b.to(y.dtype)


class _RefSwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, e, g, mod):
        ctx.mod = mod
        ctx.save_for_backward(e, g)
        return mod.swiglu_fg_kernel(e[None], g[None])[0]

    @staticmethod
    def backward(ctx, dh):
        e, g = ctx.saved_tensors
        # the reference's kernel works in place: (dh, e, g) become (h, dh * f, de); dg = dh * f
        dh, e, g = dh.contiguous().clone(), e.clone(), g.clone()
        _h, dg, de = ctx.mod.swiglu_DWf_DW_dfg_kernel(dh, e, g)
        return de, dg, None


def _rope(x, pos, cos_t, sin_t):
    d = x.shape[-1]
    c = cos_t[pos][:, None, :].to(x.dtype)
    s = sin_t[pos][:, None, :].to(x.dtype)
    x1, x2 = x[..., : d // 2], x[..., d // 2:]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1)


class BaselineRunner(nn.Module):
    """Runs ``model`` (an in-tree Llama-family ``...ForCausalLM``, optionally wrapped by the LoRA shim) on packed
    batches with library kernels.  ``runner(input_ids=, labels=, cu_seqlens=)`` returns an object with ``.loss``."""

    def __init__(self, model: nn.Module, gradient_checkpointing: bool = False):
        super().__init__()
        self.wrapped = model
        base = model.get_base_model() if hasattr(model, "get_base_model") else model
        self.base = base
        self.cfg = base.config
        self.gradient_checkpointing = gradient_checkpointing
        cuda = next(base.parameters()).is_cuda
        self.k_rms = _try("rmsnorm", "fms_acceleration_foak", "kernels.unsloth.rms_layernorm") if cuda else None
        self.k_glu = _try("swiglu", "fms_acceleration_foak", "fused_ops.unsloth_lora.swiglu") if cuda else None
        self.k_lce = _try("fused_linear_cross_entropy", "fms_acceleration_foak",
                          "fused_ops.liger_ce.fused_linear_cross_entropy_loss") if cuda else None
        try:
            from flash_attn import flash_attn_varlen_func

            self.flash = flash_attn_varlen_func if cuda else None
            _STATUS["attention"] = "flash_attn_varlen_func (installed flash-attn)" if cuda else "torch SDPA per document"
        except Exception as exc:  # pragma: no cover
            self.flash = None
            _STATUS["attention"] = f"torch SDPA per document ({type(exc).__name__})"
        self.k_moe = None
        moes = [m for m in base.modules() if m.__class__.__name__ == "ScatterMoE"]
        if moes:
            for m in moes:  # whatever happens, never this package's fused path
                m.backend = "library"
            self.k_moe = _try("moe", "fms_acceleration_moe", "utils.scattermoe_utils.khd.kernels.ops") if cuda else None
            if self.k_moe is None:
                _STATUS["moe"] = "per-expert torch.matmul + all_to_all_single (ScatterMoE library backend); " + \
                    _STATUS.get("moe", "")
            elif moes[0].expert_parallel:
                _STATUS["moe"] += " after all_to_all_single (NCCL)"

    def parameters(self, recurse: bool = True):  # the wrapped model's parameters, once
        return self.wrapped.parameters(recurse)

    # ------------------------------------------------------------------ pieces
    def _rms(self, norm, x):
        if self.k_rms is not None:
            return self.k_rms.fast_rms_layernorm(norm, x)
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + norm.variance_epsilon)).to(x.dtype) * norm.weight

    def _glu(self, e, g, act):
        if self.k_glu is not None and act in ("silu", "swiglu"):
            return _RefSwiGLU.apply(e.contiguous(), g.contiguous(), self.k_glu)
        fn = {"silu": F.silu, "gelu": F.gelu}.get(act, lambda t: F.gelu(t, approximate="tanh"))
        return fn(e) * g

    def _attention(self, a, h, pos, cos_t, sin_t, cu, max_len, cu_list):
        T = h.shape[0]
        q = _linear(a.q_proj, h).view(T, a.num_heads, a.head_dim)
        k = _linear(a.k_proj, h).view(T, a.num_kv_heads, a.head_dim)
        v = _linear(a.v_proj, h).view(T, a.num_kv_heads, a.head_dim)
        q, k = _rope(q, pos, cos_t, sin_t), _rope(k, pos, cos_t, sin_t)
        if self.flash is not None:
            o = self.flash(q, k, v, cu, cu, max_len, max_len, causal=True, softmax_scale=a.scaling)
        else:
            rep = a.num_heads // a.num_kv_heads
            outs = []
            for s, e in zip(cu_list[:-1], cu_list[1:]):
                qd = q[s:e].transpose(0, 1)[None]
                kd = k[s:e].repeat_interleave(rep, 1).transpose(0, 1)[None]
                vd = v[s:e].repeat_interleave(rep, 1).transpose(0, 1)[None]
                outs.append(F.scaled_dot_product_attention(qd, kd, vd, is_causal=True, scale=a.scaling)[0].transpose(0, 1))
            o = torch.cat(outs, 0)
        return _linear(a.o_proj, o.reshape(T, -1))

    def _layer(self, layer, x, pos, cos_t, sin_t, cu, max_len, cu_list):
        rm = self.cfg.residual_multiplier
        x = x + rm * self._attention(layer.self_attn, self._rms(layer.input_layernorm, x), pos, cos_t, sin_t, cu, max_len,
                                     cu_list)
        h = self._rms(layer.post_attention_layernorm, x)
        mlp = getattr(layer, "mlp", None)
        if mlp is not None and hasattr(mlp, "gate_proj"):
            out = _linear(mlp.down_proj, self._glu(_linear(mlp.gate_proj, h), _linear(mlp.up_proj, h), mlp.hidden_act))
        else:
            ffn = getattr(layer, "_ffn", None) or (mlp if mlp is not None else layer.block_sparse_moe)
            if self.k_moe is not None and ffn.__class__.__name__ == "ScatterMoE":
                out = self._moe(ffn, h)
            else:
                out = ffn(h)
                out = out[0] if isinstance(out, tuple) else out
        return x + rm * out

    def _moe(self, moe, h):
        """The reference's ScatterMoE forward on its own Triton kernels."""
        ops = self.k_moe
        k, El = moe.top_k, moe.num_experts_per_device
        logits = h @ moe.router.weight.t()
        w, idx = torch.topk(torch.softmax(logits.float(), dim=-1), k, dim=-1)
        w = (w / w.sum(-1, keepdim=True)).to(h.dtype)
        act = {"silu": F.silu, "gelu": F.gelu}.get(moe.activation, F.silu)
        w1, w2, w3 = moe.w1.effective_weight(), moe.w2.effective_weight(), moe.w3.effective_weight()
        if not moe.expert_parallel:
            se, ss = torch.sort(idx.flatten())
            with torch.no_grad():
                pb, eo = ops.padded_block_indices(se, moe.num_experts)
            up = ops.scattered_experts(h, w1, k, se, ss, pb, eo, grouped_out=True)
            up = act(up) * ops.scattered_experts(h, w3, k, se, ss, pb, eo, grouped_out=True)
            return ops.scattered_experts(up, w2, 1, se, ss, pb, eo, gates=w, grouped_in=True)
        from ..plugins.moe.utils.scattermoe_utils import all_to_all_gather_inputs, scatter_with_routing_weights

        rows, local_e, state = all_to_all_gather_inputs(h, idx.to(torch.int32), moe.ep_group, k, El)
        ss = torch.arange(rows.shape[0], device=h.device)
        with torch.no_grad():
            pb, eo = ops.padded_block_indices(local_e, El)
        up = ops.scattered_experts(rows, w1, 1, local_e, ss, pb, eo, grouped_in=True, grouped_out=True)
        up = act(up) * ops.scattered_experts(rows, w3, 1, local_e, ss, pb, eo, grouped_in=True, grouped_out=True)
        y = ops.scattered_experts(up, w2, 1, local_e, ss, pb, eo, grouped_in=True, grouped_out=True)
        return scatter_with_routing_weights(y, w, state).to(h.dtype)

    # ------------------------------------------------------------------ forward
    def forward(self, input_ids, labels=None, cu_seqlens=None, position_ids=None, **_):
        from ..models.llama import CausalLMOutput

        base, cfg = self.base, self.cfg
        ids = input_ids.reshape(-1)
        T = ids.numel()
        dev = ids.device
        if cu_seqlens is None:
            if position_ids is not None:
                starts = torch.nonzero(position_ids.reshape(-1) == 0).reshape(-1)
                cu_seqlens = torch.cat([starts, starts.new_tensor([T])]).to(torch.int32)
            else:
                S = input_ids.shape[-1]
                cu_seqlens = torch.arange(0, T + 1, S, device=dev, dtype=torch.int32)
        cu = cu_seqlens.to(device=dev, dtype=torch.int32)
        idx = torch.arange(T, device=dev)
        doc = torch.searchsorted(cu.long(), idx, right=True) - 1
        pos = idx - cu.long()[doc]
        lens = cu[1:] - cu[:-1]
        if self.flash is not None:
            max_len, cu_list = int(lens.max().item()), None  # flash-attn wants the longest document as a host integer
        else:
            cu_list = [int(c) for c in cu.tolist()]
            max_len = max(b - a for a, b in zip(cu_list[:-1], cu_list[1:]))
        cos_t, sin_t = base.model.rope(dev, max(max_len, 1))
        x = base.model.embed_tokens(ids)
        if cfg.embedding_multiplier != 1.0:
            x = x * cfg.embedding_multiplier
        for layer in base.model.layers:
            if self.gradient_checkpointing and torch.is_grad_enabled() and x.requires_grad:
                from torch.utils.checkpoint import checkpoint

                x = checkpoint(self._layer, layer, x, pos, cos_t, sin_t, cu, max_len, cu_list, use_reentrant=False)
            else:
                x = self._layer(layer, x, pos, cos_t, sin_t, cu, max_len, cu_list)
        x = self._rms(base.model.norm, x)
        if cfg.logits_scaling != 1.0:
            x = x / cfg.logits_scaling
        loss = None
        if labels is not None:
            flat = labels.reshape(-1)
            shift = torch.cat([flat[1:], flat.new_full((1,), IGNORE)])
            w = base.lm_head.weight
            if self.k_lce is not None:
                loss = self.k_lce.LigerFusedLinearCrossEntropyFunction.apply(x, w, shift, None, IGNORE, 0.0, "mean")
            else:
                # chunked so that the [T, vocab] logits never exist as a whole
                n = (shift != IGNORE).sum().clamp(min=1)
                total = x.new_zeros((), dtype=torch.float32)
                for s in range(0, T, 4096):
                    logits = (x[s:s + 4096] @ w.t()).float()
                    total = total + F.cross_entropy(logits, shift[s:s + 4096], ignore_index=IGNORE, reduction="sum")
                loss = total / n
        return CausalLMOutput(loss=loss, logits=None)
