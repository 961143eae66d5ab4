"""Mixtral-style decoder: Llama attention + top-k mixture of experts with one module per expert in the Hugging Face
layout (``block_sparse_moe.gate.weight [E, H]``, ``block_sparse_moe.experts.<i>.{w1,w2,w3}.weight``; ``w1`` gate,
``w3`` up, ``w2`` down).  This is the "sharded" expert layout the ScatterMoE conversion handles next to GraniteMoe's
fused one (fms_acceleration_moe/utils/scattermoe_constants.py:72-95 of the reference).  The eager block loops over
the experts; the ScatterMoE plugin swaps it for the grouped-GEMM module."""
from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import nn

from .config import DecoderConfig
from .llama import LlamaDecoderLayer, LlamaForCausalLM, LlamaModel


class MixtralBlockSparseTop2MLP(nn.Module):
    def __init__(self, cfg: DecoderConfig):
        super().__init__()
        H, I = cfg.hidden_size, cfg.moe_intermediate_size or cfg.intermediate_size
        self.w1 = nn.Linear(H, I, bias=False)
        self.w2 = nn.Linear(I, H, bias=False)
        self.w3 = nn.Linear(H, I, bias=False)

    def forward(self, x):
        return self.w2(F.silu(self.w1(x)) * self.w3(x))


class MixtralSparseMoeBlock(nn.Module):
    def __init__(self, cfg: DecoderConfig):
        super().__init__()
        self.hidden_dim = cfg.hidden_size
        self.ffn_dim = cfg.moe_intermediate_size or cfg.intermediate_size
        self.num_experts, self.top_k = cfg.num_local_experts, cfg.num_experts_per_tok
        self.gate = nn.Linear(self.hidden_dim, self.num_experts, bias=False)
        self.experts = nn.ModuleList([MixtralBlockSparseTop2MLP(cfg) for _ in range(self.num_experts)])

    def forward(self, x):
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        logits = self.gate(x2)
        probs = torch.softmax(logits.float(), dim=-1)
        w, idx = torch.topk(probs, self.top_k, dim=-1)
        w = (w / w.sum(-1, keepdim=True)).to(x.dtype)
        out = torch.zeros_like(x2)
        for e, expert in enumerate(self.experts):
            tok, slot = torch.nonzero(idx == e, as_tuple=True)
            if tok.numel():
                out.index_add_(0, tok, expert(x2[tok]) * w[tok, slot][:, None])
        return out.view(shape), logits


class MixtralDecoderLayer(LlamaDecoderLayer):
    def _build_mlp(self, cfg):
        return None

    def __init__(self, cfg: DecoderConfig, layer_idx: int):
        super().__init__(cfg, layer_idx)
        self.block_sparse_moe = MixtralSparseMoeBlock(cfg)

    def forward(self, x, pos, cos_t, sin_t, cu_seqlens):
        x = x + self.self_attn(self.input_layernorm(x), pos, cos_t, sin_t, cu_seqlens)
        moe_out, _ = self.block_sparse_moe(self.post_attention_layernorm(x))
        return x + moe_out


class MixtralModel(LlamaModel):
    layer_cls = MixtralDecoderLayer


class MixtralForCausalLM(LlamaForCausalLM):
    model_cls = MixtralModel
