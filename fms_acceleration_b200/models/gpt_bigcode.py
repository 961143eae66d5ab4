"""GPTBigCode (santacoder / starcoder) decoder with Hugging Face module names: ``transformer.wte``, ``transformer.wpe``
(learned absolute positions), blocks ``transformer.h.<i>.{ln_1, attn.{c_attn, c_proj}, ln_2, mlp.{c_fc, c_proj}}``,
``transformer.ln_f``, tied ``lm_head``.  Multi-query attention (one key/value head), LayerNorm with bias, tanh-GELU MLP.
The reference benchmarks this family (scripts/benchmarks/scenarios.yaml:44,91) and patches its loss and LoRA layers
(fms_acceleration_foak/models/gpt_bigcode.py).  Attention over packed documents uses the in-tree varlen kernel on a
GPU and per-document SDPA elsewhere."""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as F
from torch import nn

from ..ops import cross_entropy as CE
from .config import DecoderConfig
from .generation import GenerationMixin
from .llama import CausalLMOutput, _init_weights, _run_layer


class GPTBigCodeAttention(nn.Module):
    def __init__(self, cfg: DecoderConfig, layer_idx: int):
        super().__init__()
        self.num_heads, self.head_dim = cfg.num_attention_heads, cfg.head_dim
        self.kv_heads = cfg.num_key_value_heads  # 1 for multi-query
        H = cfg.hidden_size
        self.c_attn = nn.Linear(H, H + 2 * self.kv_heads * self.head_dim)
        self.c_proj = nn.Linear(H, H)
        self.scaling = 1.0 / math.sqrt(self.head_dim)

    def forward(self, x, cu):
        T, H = x.shape
        qkv = self.c_attn(x)
        kvd = self.kv_heads * self.head_dim
        q, k, v = qkv[:, :H], qkv[:, H:H + kvd], qkv[:, H + kvd:]
        if x.is_cuda and x.dtype in (torch.bfloat16, torch.float16) and self.head_dim in (64, 128):
            from ..ops.attention import doc_bounds_from_cu_seqlens, varlen_attention

            cu_t = torch.as_tensor(cu, device=x.device, dtype=torch.int32)
            ds, de = doc_bounds_from_cu_seqlens(cu_t, T)
            o = varlen_attention(q.reshape(T, self.num_heads, self.head_dim), k.reshape(T, self.kv_heads, self.head_dim),
                                 v.reshape(T, self.kv_heads, self.head_dim), ds, de, self.scaling)
            return self.c_proj(o.reshape(T, H))
        q = q.view(T, self.num_heads, self.head_dim)
        k = k.view(T, self.kv_heads, self.head_dim)
        v = v.view(T, self.kv_heads, self.head_dim)
        rep = self.num_heads // self.kv_heads
        outs = []
        for s, e in zip(cu[:-1], cu[1:]):
            qd = q[s:e].transpose(0, 1).unsqueeze(0)
            kd = k[s:e].repeat_interleave(rep, dim=1).transpose(0, 1).unsqueeze(0)
            vd = v[s:e].repeat_interleave(rep, dim=1).transpose(0, 1).unsqueeze(0)
            od = F.scaled_dot_product_attention(qd, kd, vd, is_causal=True, scale=self.scaling)
            outs.append(od.squeeze(0).transpose(0, 1).reshape(e - s, -1))
        return self.c_proj(torch.cat(outs, dim=0))


class GPTBigCodeMLP(nn.Module):
    def __init__(self, cfg: DecoderConfig):
        super().__init__()
        self.c_fc = nn.Linear(cfg.hidden_size, cfg.intermediate_size)
        self.c_proj = nn.Linear(cfg.intermediate_size, cfg.hidden_size)

    def forward(self, x):
        return self.c_proj(F.gelu(self.c_fc(x), approximate="tanh"))


class GPTBigCodeBlock(nn.Module):
    def __init__(self, cfg: DecoderConfig, layer_idx: int):
        super().__init__()
        self.ln_1 = nn.LayerNorm(cfg.hidden_size, eps=cfg.rms_norm_eps)
        self.attn = GPTBigCodeAttention(cfg, layer_idx)
        self.ln_2 = nn.LayerNorm(cfg.hidden_size, eps=cfg.rms_norm_eps)
        self.mlp = GPTBigCodeMLP(cfg)

    def forward(self, x, cu):
        x = x + self.attn(self.ln_1(x), cu)
        return x + self.mlp(self.ln_2(x))


class GPTBigCodeModel(nn.Module):
    def __init__(self, cfg: DecoderConfig, layer_hook=None):
        super().__init__()
        self.cfg = cfg
        self.wte = nn.Embedding(cfg.vocab_size, cfg.hidden_size)
        self.wpe = nn.Embedding(cfg.max_position_embeddings, cfg.hidden_size)
        for emb in (self.wte, self.wpe):
            nn.init.normal_(emb.weight, 0.0, cfg.initializer_range)
        blocks = []
        for i in range(cfg.num_hidden_layers):
            blk = GPTBigCodeBlock(cfg, i)
            blk.apply(lambda m: _init_weights(m, cfg.initializer_range))
            if layer_hook is not None:
                blk = layer_hook(blk) or blk
            blocks.append(blk)
        self.h = nn.ModuleList(blocks)
        self.ln_f = nn.LayerNorm(cfg.hidden_size, eps=cfg.rms_norm_eps)

    def forward(self, input_ids, position_ids=None, cu_seqlens=None):
        B, S = input_ids.shape
        T = B * S
        dev = input_ids.device
        if cu_seqlens is not None:
            cu = [int(c) for c in cu_seqlens.tolist()]
            cu_t = torch.as_tensor(cu, device=dev)
            idx = torch.arange(T, device=dev)
            pos = idx - cu_t[torch.searchsorted(cu_t, idx, right=True) - 1]
        else:
            if position_ids is None:
                position_ids = torch.arange(S, device=dev).expand(B, S)
            pos = position_ids.reshape(-1)
            cu = torch.nonzero(pos == 0).reshape(-1).tolist() + [T]
        x = self.wte(input_ids.reshape(-1)) + self.wpe(pos)
        for blk in self.h:
            x = _run_layer(self, blk, x, cu)
        return self.ln_f(x)


class GPTBigCodeForCausalLM(GenerationMixin, nn.Module):
    def __init__(self, cfg: DecoderConfig, layer_hook=None):
        super().__init__()
        self.config = cfg
        self.transformer = GPTBigCodeModel(cfg, layer_hook)
        self.lm_head = nn.Linear(cfg.hidden_size, cfg.vocab_size, bias=False)
        self.lm_head.weight = self.transformer.wte.weight  # always tied in this family
        self.fast_loss = False

    def get_input_embeddings(self):
        return self.transformer.wte

    def get_output_embeddings(self):
        return self.lm_head

    def gradient_checkpointing_enable(self, gradient_checkpointing_kwargs=None, **kwargs):
        self.transformer.gradient_checkpointing = True

    def gradient_checkpointing_disable(self):
        self.transformer.gradient_checkpointing = False

    def enable_input_require_grads(self):
        self.transformer.wte.register_forward_hook(lambda m, i, o: o.requires_grad_(True))

    def enable_fused(self, fast_loss="fused_ce_liger"):
        self.fast_loss = fast_loss
        return self

    def forward(self, input_ids, labels=None, position_ids=None, attention_mask=None, cu_seqlens=None,
                num_items_in_batch=None, return_logits: Optional[bool] = None, **kwargs):
        hidden = self.transformer(input_ids, position_ids=position_ids, cu_seqlens=cu_seqlens)
        loss = logits = None
        if labels is not None:
            flat = labels.reshape(-1)
            shift = torch.cat([flat[1:], flat.new_full((1,), CE.IGNORE_INDEX)])
            if input_ids.shape[0] > 1:
                S = input_ids.shape[1]
                shift = shift.clone()
                shift[S - 1:: S] = CE.IGNORE_INDEX
            if hidden.is_cuda and self.fast_loss == "fused_ce_liger" and not return_logits:
                loss = CE.fused_linear_cross_entropy(hidden, self.lm_head.weight, shift, num_items=num_items_in_batch)
                return CausalLMOutput(loss=loss, logits=None)
            logits = self.lm_head(hidden)
            per = CE.fast_cross_entropy_loss(logits, shift) if (self.fast_loss and logits.is_cuda) else \
                CE.cross_entropy_ref(logits, shift)
            n = num_items_in_batch if num_items_in_batch is not None else (shift != CE.IGNORE_INDEX).sum().clamp(min=1)
            loss = per.sum() / n
        else:
            logits = self.lm_head(hidden)
        return CausalLMOutput(loss=loss, logits=logits.view(*input_ids.shape, -1))
