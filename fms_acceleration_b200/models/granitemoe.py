"""GraniteMoe-style decoder: Llama attention + a top-k mixture-of-experts feed-forward with fused expert weights
in the Hugging Face layout (``block_sparse_moe.input_linear.weight [E, 2I, H]``, ``output_linear.weight [E, H, I]``,
``router.layer.weight [E, H]``).  The eager block below loops over experts (the unaccelerated baseline); the
ScatterMoE plugin swaps it for the grouped-GEMM module."""
from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import nn

from .config import DecoderConfig
from .llama import LlamaDecoderLayer, LlamaForCausalLM, LlamaModel


class GraniteMoeParallelExperts(nn.Module):
    def __init__(self, num_experts: int, input_size: int, output_size: int):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(num_experts, output_size, input_size))
        self.num_experts, self.input_size, self.output_size = num_experts, input_size, output_size


class GraniteMoeTopKGating(nn.Module):
    def __init__(self, input_size: int, num_experts: int, top_k: int):
        super().__init__()
        self.layer = nn.Linear(input_size, num_experts, bias=False)
        self.num_experts, self.top_k = num_experts, top_k


class GraniteMoeMoE(nn.Module):
    """Reference (loop-over-experts) implementation."""

    def __init__(self, cfg: DecoderConfig):
        super().__init__()
        self.input_size = cfg.hidden_size
        self.hidden_size = cfg.moe_intermediate_size or cfg.intermediate_size
        self.num_experts, self.top_k = cfg.num_local_experts, cfg.num_experts_per_tok
        self.input_linear = GraniteMoeParallelExperts(self.num_experts, self.input_size, 2 * self.hidden_size)
        self.output_linear = GraniteMoeParallelExperts(self.num_experts, self.hidden_size, self.input_size)
        self.router = GraniteMoeTopKGating(self.input_size, self.num_experts, self.top_k)
        self.hidden_act = cfg.hidden_act
        for p in (self.input_linear.weight, self.output_linear.weight):
            nn.init.normal_(p, 0.0, cfg.initializer_range)

    def forward(self, x):
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        logits = self.router.layer(x2)
        probs = torch.softmax(logits.float(), dim=-1)
        w, idx = torch.topk(probs, self.top_k, dim=-1)
        w = (w / w.sum(-1, keepdim=True)).to(x.dtype)
        out = torch.zeros_like(x2)
        I = self.hidden_size
        for e in range(self.num_experts):
            tok, slot = torch.nonzero(idx == e, as_tuple=True)
            if tok.numel() == 0:
                continue
            h = x2[tok] @ self.input_linear.weight[e].t()
            h = F.silu(h[:, :I]) * h[:, I:]
            out.index_add_(0, tok, (h @ self.output_linear.weight[e].t()) * w[tok, slot][:, None])
        return out.view(shape), logits


class GraniteMoeDecoderLayer(LlamaDecoderLayer):
    def _build_mlp(self, cfg):
        return None

    def __init__(self, cfg: DecoderConfig, layer_idx: int):
        super().__init__(cfg, layer_idx)
        self.block_sparse_moe = GraniteMoeMoE(cfg)

    def forward(self, x, pos, cos_t, sin_t, cu_seqlens):
        rm = self.cfg.residual_multiplier
        # x + rm * y as ONE element-wise kernel (add with alpha), not a multiply followed by an add
        x = torch.add(x, self.self_attn(self.input_layernorm(x), pos, cos_t, sin_t, cu_seqlens), alpha=rm)
        moe_out, _ = self.block_sparse_moe(self.post_attention_layernorm(x))
        return torch.add(x, moe_out, alpha=rm)


class GraniteMoeModel(LlamaModel):
    layer_cls = GraniteMoeDecoderLayer


class GraniteMoeForCausalLM(LlamaForCausalLM):
    model_cls = GraniteMoeModel


# ------------------------------------------------------------------------------ GraniteMoeShared
class GraniteMoeSharedMLP(nn.Module):
    """Dense SwiGLU branch that every token takes besides its routed experts (``shared_mlp.input_linear [2*Is, H]``,
    ``shared_mlp.output_linear [H, Is]`` as in the Hugging Face GraniteMoeShared checkpoints)."""

    def __init__(self, cfg: DecoderConfig):
        super().__init__()
        self.input_linear = nn.Linear(cfg.hidden_size, 2 * cfg.shared_intermediate_size, bias=False)
        self.output_linear = nn.Linear(cfg.shared_intermediate_size, cfg.hidden_size, bias=False)

    def forward(self, x):
        g, u = self.input_linear(x).chunk(2, dim=-1)
        return self.output_linear(F.silu(g) * u)


class GraniteMoeSharedMoE(GraniteMoeMoE):
    pass


class GraniteMoeSharedDecoderLayer(GraniteMoeDecoderLayer):
    def __init__(self, cfg: DecoderConfig, layer_idx: int):
        super().__init__(cfg, layer_idx)
        self.block_sparse_moe = GraniteMoeSharedMoE(cfg)
        self.shared_mlp = GraniteMoeSharedMLP(cfg) if cfg.shared_intermediate_size else None

    def _ffn(self, y):
        out = self.block_sparse_moe(y)
        out = out[0] if isinstance(out, tuple) else out
        if self.shared_mlp is not None:
            out = out + self.shared_mlp(y)
        return out

    def forward(self, x, pos, cos_t, sin_t, cu_seqlens):
        rm = self.cfg.residual_multiplier
        x = torch.add(x, self.self_attn(self.input_layernorm(x), pos, cos_t, sin_t, cu_seqlens), alpha=rm)
        return torch.add(x, self._ffn(self.post_attention_layernorm(x)), alpha=rm)


class GraniteMoeSharedModel(LlamaModel):
    layer_cls = GraniteMoeSharedDecoderLayer


class GraniteMoeSharedForCausalLM(LlamaForCausalLM):
    model_cls = GraniteMoeSharedModel
