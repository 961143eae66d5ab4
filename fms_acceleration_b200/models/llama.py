"""Llama / Mistral / Granite style decoder with HF-compatible module names.

Two execution paths share the same parameters:

* the *eager* path is plain PyTorch (runs on CPU; the oracle for the fused path and the model of the
  CPU plumbing configuration);
* the *fused* path runs on packed tokens ``[T, H]`` through :mod:`fms_acceleration_b200.ops.fused_layer`
  (tcgen05 GEMMs with fused LoRA, in-place RoPE, varlen attention, fused norms, chunked linear+CE).  It is
  switched on per model by :func:`enable_fused`, which is what the fused-ops plugin does in ``augmentation``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn.functional as F
from torch import nn

from ..ops import cross_entropy as CE
from ..ops import rmsnorm as RN
from ..ops.rope import rope_ref, rope_tables
from .config import DecoderConfig
from .generation import GenerationMixin


@dataclass
class CausalLMOutput:
    loss: Optional[torch.Tensor] = None
    logits: Optional[torch.Tensor] = None
    hidden_states: Optional[torch.Tensor] = None
    aux_loss: Optional[torch.Tensor] = None
    router_logits: Optional[tuple] = None

    def __getitem__(self, k):
        return getattr(self, k) if isinstance(k, str) else (self.loss, self.logits)[k]


def _init_weights(m, std):
    if isinstance(m, nn.Linear):
        nn.init.normal_(m.weight, 0.0, std)
        if m.bias is not None:
            nn.init.zeros_(m.bias)
    elif isinstance(m, nn.Embedding):
        nn.init.normal_(m.weight, 0.0, std)


class LlamaRMSNorm(nn.Module):
    def __init__(self, hidden_size: int, eps: float = 1e-6):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden_size))
        self.variance_epsilon = eps

    def forward(self, x):
        y, _ = RN.rmsnorm_ref(x, self.weight, self.variance_epsilon)
        return y


class LlamaMLP(nn.Module):
    def __init__(self, cfg: DecoderConfig):
        super().__init__()
        H, I = cfg.hidden_size, cfg.intermediate_size
        self.gate_proj = nn.Linear(H, I, bias=False)
        self.up_proj = nn.Linear(H, I, bias=False)
        self.down_proj = nn.Linear(I, H, bias=False)
        self.hidden_act = cfg.hidden_act

    def forward(self, x):
        act = {"silu": F.silu, "gelu": F.gelu}.get(self.hidden_act, lambda t: F.gelu(t, approximate="tanh"))
        return self.down_proj(act(self.gate_proj(x)) * self.up_proj(x))


class LlamaAttention(nn.Module):
    def __init__(self, cfg: DecoderConfig, layer_idx: int):
        super().__init__()
        self.cfg = cfg
        self.layer_idx = layer_idx
        self.num_heads, self.num_kv_heads, self.head_dim = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        H = cfg.hidden_size
        self.q_proj = nn.Linear(H, self.num_heads * self.head_dim, bias=False)
        self.k_proj = nn.Linear(H, self.num_kv_heads * self.head_dim, bias=False)
        self.v_proj = nn.Linear(H, self.num_kv_heads * self.head_dim, bias=False)
        self.o_proj = nn.Linear(self.num_heads * self.head_dim, H, bias=False)
        self.scaling = cfg.attention_multiplier if cfg.attention_multiplier is not None else 1.0 / math.sqrt(self.head_dim)

    def forward(self, x, pos, cos_t, sin_t, cu_seqlens):
        # x: [T, H] packed
        T = x.shape[0]
        q = self.q_proj(x).view(T, self.num_heads, self.head_dim)
        k = self.k_proj(x).view(T, self.num_kv_heads, self.head_dim)
        v = self.v_proj(x).view(T, self.num_kv_heads, self.head_dim)
        q = rope_ref(q, pos, cos_t, sin_t)
        k = rope_ref(k, pos, cos_t, sin_t)
        rep = self.num_heads // self.num_kv_heads
        outs = []
        for s, e in zip(cu_seqlens[:-1], cu_seqlens[1:]):
            qd = q[s:e].transpose(0, 1).unsqueeze(0)
            kd = k[s:e].repeat_interleave(rep, dim=1).transpose(0, 1).unsqueeze(0)
            vd = v[s:e].repeat_interleave(rep, dim=1).transpose(0, 1).unsqueeze(0)
            od = F.scaled_dot_product_attention(qd, kd, vd, is_causal=True, scale=self.scaling)
            outs.append(od.squeeze(0).transpose(0, 1).reshape(e - s, -1))
        return self.o_proj(torch.cat(outs, dim=0))


class LlamaDecoderLayer(nn.Module):
    def __init__(self, cfg: DecoderConfig, layer_idx: int):
        super().__init__()
        self.cfg = cfg
        self.layer_idx = layer_idx
        self.self_attn = LlamaAttention(cfg, layer_idx)
        mlp = self._build_mlp(cfg)
        if mlp is not None:
            self.mlp = mlp
        self.input_layernorm = LlamaRMSNorm(cfg.hidden_size, cfg.rms_norm_eps)
        self.post_attention_layernorm = LlamaRMSNorm(cfg.hidden_size, cfg.rms_norm_eps)
        self._fused_specs = None

    def _build_mlp(self, cfg):
        return LlamaMLP(cfg)

    # eager
    def forward(self, x, pos, cos_t, sin_t, cu_seqlens):
        rm = self.cfg.residual_multiplier
        x = torch.add(x, self.self_attn(self.input_layernorm(x), pos, cos_t, sin_t, cu_seqlens), alpha=rm)
        x = torch.add(x, self.mlp(self.post_attention_layernorm(x)), alpha=rm)
        return x

    # fused
    def fused_specs(self):
        if self._fused_specs is None:
            from ..ops.fused_layer import AttentionBlockSpec, MLPBlockSpec

            a = self.self_attn
            tag = f"L{self.layer_idx}"
            attn = AttentionBlockSpec(self.input_layernorm, a.q_proj, a.k_proj, a.v_proj, a.o_proj, a.num_heads,
                                      a.num_kv_heads, a.head_dim, tag, a.scaling, self.cfg.residual_multiplier)
            mlp = None
            if isinstance(getattr(self, "mlp", None), LlamaMLP):
                m = self.mlp
                mlp = MLPBlockSpec(self.post_attention_layernorm, m.gate_proj, m.up_proj, m.down_proj, m.hidden_act,
                                   tag, self.cfg.residual_multiplier)
            self._fused_specs = (attn, mlp)
        return self._fused_specs

    def forward_fused(self, x, batch):
        from ..ops.fused_layer import attention_block, mlp_block

        attn, mlp = self.fused_specs()
        h = attention_block(x, attn, batch)
        if mlp is not None:
            return mlp_block(h, mlp)
        y = RN.rmsnorm(h, self.post_attention_layernorm.weight, self.post_attention_layernorm.variance_epsilon)
        ffn = getattr(self, "_ffn", None) or (self.mlp if hasattr(self, "mlp") else self.block_sparse_moe)
        out = ffn(y)
        if isinstance(out, tuple):
            out = out[0]
        return torch.add(h, out, alpha=self.cfg.residual_multiplier)


def _run_layer(model, fn, x, *args):
    """One decoder layer, under activation checkpointing when the model asks for it (the reference benchmarks run
    with it on, scripts/benchmarks/defaults.yaml:15): only the layer input is kept and the layer runs a second time
    in backward."""
    if getattr(model, "gradient_checkpointing", False) and model.training and torch.is_grad_enabled() and x.requires_grad:
        from torch.utils.checkpoint import checkpoint

        return checkpoint(fn, x, *args, use_reentrant=False)
    return fn(x, *args)


class LlamaModel(nn.Module):
    layer_cls = LlamaDecoderLayer

    def __init__(self, cfg: DecoderConfig, layer_hook=None):
        super().__init__()
        self.cfg = cfg
        self.embed_tokens = nn.Embedding(cfg.vocab_size, cfg.hidden_size)
        nn.init.normal_(self.embed_tokens.weight, 0.0, cfg.initializer_range)
        layers = []
        for i in range(cfg.num_hidden_layers):
            layer = self.layer_cls(cfg, i)
            layer.apply(lambda m: _init_weights(m, cfg.initializer_range))
            if layer_hook is not None:
                # e.g. quantise the layer right away so a large model never exists in 16 bits as a whole
                layer = layer_hook(layer) or layer
            layers.append(layer)
        self.layers = nn.ModuleList(layers)
        self.norm = LlamaRMSNorm(cfg.hidden_size, cfg.rms_norm_eps)
        self._rope = None
        self.fused = False
        self.gradient_checkpointing = False  # recompute every decoder layer in backward instead of keeping its activations

    def rope(self, device, max_pos: int):
        if self._rope is None or self._rope[0].device != torch.device(device) or self._rope[0].shape[0] < max_pos:
            n = max(max_pos, min(self.cfg.max_position_embeddings, 8192))
            self._rope = rope_tables(self.cfg.head_dim, n, self.cfg.rope_theta, device)
        return self._rope

    def forward(self, input_ids, position_ids=None, cu_seqlens=None, max_seqlen=None):
        """Returns packed hidden states [T, H] (T = number of tokens in the batch)."""
        B, S = input_ids.shape
        T = B * S
        dev = input_ids.device
        if position_ids is None and cu_seqlens is None:
            position_ids = torch.arange(S, device=dev).expand(B, S)
        x = self.embed_tokens(input_ids.reshape(-1))
        if self.cfg.embedding_multiplier != 1.0:
            x = x * self.cfg.embedding_multiplier
        max_pos = max_seqlen or (S if B > 1 or position_ids is None else T)
        cos_t, sin_t = self.rope(dev, max(max_pos, S, 1) if cu_seqlens is None else max(max_pos, T))
        if self.fused and x.is_cuda:
            from ..ops.fused_layer import PackedBatch

            if cu_seqlens is not None:
                batch = PackedBatch.from_cu_seqlens(cu_seqlens, T, cos_t, sin_t)
            else:
                batch = PackedBatch.from_position_ids(position_ids, cos_t, sin_t)
            x = x.contiguous()
            for layer in self.layers:
                x = _run_layer(self, layer.forward_fused, x, batch)
            return RN.rmsnorm(x, self.norm.weight, self.norm.variance_epsilon)
        # eager
        if cu_seqlens is None:
            flat = position_ids.reshape(-1)
            starts = torch.nonzero(flat == 0).reshape(-1).tolist()
            cu = starts + [T]
            pos = flat
        else:
            cu = cu_seqlens.tolist()
            cu_t = torch.as_tensor(cu, device=dev)
            idx = torch.arange(T, device=dev)
            doc = torch.searchsorted(cu_t, idx, right=True) - 1
            pos = idx - cu_t[doc]
        for layer in self.layers:
            x = _run_layer(self, layer, x, pos, cos_t, sin_t, cu)
        return self.norm(x)


class LlamaForCausalLM(GenerationMixin, nn.Module):
    model_cls = LlamaModel

    def __init__(self, cfg: DecoderConfig, layer_hook=None):
        super().__init__()
        self.config = cfg
        self.model = self.model_cls(cfg, layer_hook=layer_hook)
        self.lm_head = nn.Linear(cfg.hidden_size, cfg.vocab_size, bias=False)
        if cfg.tie_word_embeddings:
            self.lm_head.weight = self.model.embed_tokens.weight
        else:
            nn.init.normal_(self.lm_head.weight, 0.0, cfg.initializer_range)
        self.fast_loss = False  # False | True | "fused_ce_liger"

    # HF-style helpers
    def get_input_embeddings(self):
        return self.model.embed_tokens

    def get_output_embeddings(self):
        return self.lm_head

    def gradient_checkpointing_enable(self, gradient_checkpointing_kwargs=None, **kwargs):
        self.model.gradient_checkpointing = True

    def gradient_checkpointing_disable(self):
        self.model.gradient_checkpointing = False

    def enable_input_require_grads(self):
        self.model.embed_tokens.register_forward_hook(lambda m, i, o: o.requires_grad_(True))

    def enable_fused(self, fast_loss="fused_ce_liger"):
        self.model.fused = True
        self.fast_loss = fast_loss
        return self

    def forward(self, input_ids, labels=None, position_ids=None, attention_mask=None, cu_seqlens=None,
                max_seqlen=None, num_items_in_batch=None, return_logits: Optional[bool] = None, **kwargs):
        hidden = self.model(input_ids, position_ids=position_ids, cu_seqlens=cu_seqlens, max_seqlen=max_seqlen)
        T = hidden.shape[0]
        scale = 1.0 / self.config.logits_scaling if self.config.logits_scaling != 1.0 else 1.0
        want_logits = return_logits if return_logits is not None else (labels is None or not self.fast_loss == "fused_ce_liger")
        loss = logits = None
        if labels is not None:
            flat_labels = labels.reshape(-1)
            shift_labels = torch.cat([flat_labels[1:], flat_labels.new_full((1,), CE.IGNORE_INDEX)])
            if input_ids.shape[0] > 1:
                # rows of a padded batch are independent sequences: never predict across a row boundary
                S = input_ids.shape[1]
                shift_labels = shift_labels.clone()
                shift_labels[S - 1:: S] = CE.IGNORE_INDEX
            cp = getattr(self, "cp", None)
            if cp is not None:
                # context parallelism (hybrid models): this rank holds one slice of one sequence.  Its last position
                # predicts the first token of the next rank's slice, and the mean runs over the tokens of all ranks.
                shift_labels = cp.shift_labels(flat_labels)
                if num_items_in_batch is None:
                    num_items_in_batch = cp.global_count(shift_labels != CE.IGNORE_INDEX).reshape(())
        if labels is not None and self.fast_loss == "fused_ce_liger" and hidden.is_cuda:
            h = hidden if scale == 1.0 else hidden * scale
            loss = CE.fused_linear_cross_entropy(h, self.lm_head.weight, shift_labels, num_items=num_items_in_batch)
            want_logits = bool(return_logits)
        if want_logits or (labels is not None and loss is None):
            if hidden.is_cuda and hidden.dtype in (torch.bfloat16, torch.float16) and self.model.fused:
                from ..nn.linear4bit import _QuantMatmul  # frozen-weight matmul (dx only)
                from ..ops.gemm import gemm

                if self.lm_head.weight.requires_grad:
                    logits = _DenseLinear.apply(hidden, self.lm_head.weight)
                else:
                    logits = _QuantMatmul.apply(hidden, self.lm_head.weight)
            else:
                logits = self.lm_head(hidden)
            if scale != 1.0:
                logits = logits * scale
            if labels is not None and loss is None:
                if self.fast_loss and logits.is_cuda:
                    per_tok = CE.fast_cross_entropy_loss(logits, shift_labels)
                else:
                    per_tok = CE.cross_entropy_ref(logits, shift_labels)
                n = num_items_in_batch if num_items_in_batch is not None else (shift_labels != CE.IGNORE_INDEX).sum().clamp(min=1)
                loss = per_tok.sum() / n
            logits = logits.view(*input_ids.shape, -1)
        return CausalLMOutput(loss=loss, logits=logits if want_logits else None)


class _DenseLinear(torch.autograd.Function):
    """y = x W^T with trainable dense W on the tcgen05 GEMM (dx and dW)."""

    @staticmethod
    def forward(ctx, x, w):
        from ..ops.gemm import gemm

        ctx.save_for_backward(x, w)
        return gemm(x, w)

    @staticmethod
    def backward(ctx, dy):
        from ..ops.gemm import gemm

        x, w = ctx.saved_tensors
        dy = dy.contiguous()
        dx = gemm(dy, w, b_mn=True) if ctx.needs_input_grad[0] else None
        dw = gemm(dy, x, a_mn=True, b_mn=True, out_dtype=torch.float32).to(w.dtype) if ctx.needs_input_grad[1] else None
        return dx, dw


class MistralForCausalLM(LlamaForCausalLM):
    pass


class GraniteForCausalLM(LlamaForCausalLM):
    pass
