"""GraniteMoeHybrid-style decoder: every layer is either a Mamba2 mixer or an attention block (``layer_types``),
followed by the GraniteMoeShared feed-forward (routed experts + shared dense branch).  Module names follow the
Hugging Face layout (``layers.<i>.mamba`` / ``layers.<i>.self_attn``, ``block_sparse_moe``, ``shared_mlp``); the
reference lists the family among the architectures of its ScatterMoE, fast-kernel and mamba-cp plugins
(fms_acceleration_moe/utils/scattermoe_constants.py, fms_acceleration_mcp/framework_plugin_mcp.py:27-31).
Attention layers carry no rotary embedding (position information comes from the Mamba layers)."""
from __future__ import annotations

import torch
from torch import nn

from .config import DecoderConfig
from .granitemoe import GraniteMoeMoE, GraniteMoeSharedMLP
from .llama import _run_layer, LlamaAttention, LlamaForCausalLM, LlamaRMSNorm, _init_weights
from .mamba2 import Mamba2Mixer


class GraniteMoeHybridMoE(GraniteMoeMoE):
    pass


class GraniteMoeHybridDecoderLayer(nn.Module):
    def __init__(self, cfg: DecoderConfig, layer_idx: int):
        super().__init__()
        self.cfg = cfg
        self.layer_idx = layer_idx
        self.layer_type = cfg.layer_types[layer_idx] if cfg.layer_types else "mamba"
        if self.layer_type == "mamba":
            self.mamba = Mamba2Mixer(cfg, layer_idx)
        else:
            self.self_attn = LlamaAttention(cfg, layer_idx)
        self.input_layernorm = LlamaRMSNorm(cfg.hidden_size, cfg.rms_norm_eps)
        self.post_attention_layernorm = LlamaRMSNorm(cfg.hidden_size, cfg.rms_norm_eps)
        self.block_sparse_moe = GraniteMoeHybridMoE(cfg) if cfg.num_local_experts else None
        self.shared_mlp = GraniteMoeSharedMLP(cfg) if cfg.shared_intermediate_size else None

    def forward(self, x, pos, cos_t, sin_t, cu):
        rm = self.cfg.residual_multiplier
        h = self.input_layernorm(x)
        if self.layer_type == "mamba":
            # one scan per packed document so that no state leaks across a document boundary
            mix = torch.cat([self.mamba(h[s:e]) for s, e in zip(cu[:-1], cu[1:])], dim=0) if len(cu) > 2 else self.mamba(h)
        elif getattr(self, "cp", None) is not None:
            # context parallelism: this rank holds one slice of one sequence; keys and values of the earlier slices
            # come over the group (this family's attention layers use no positional embedding)
            from ..parallel.context_parallel import cp_attention

            a, T = self.self_attn, h.shape[0]
            q = a.q_proj(h).view(T, a.num_heads, a.head_dim)
            k = a.k_proj(h).view(T, a.num_kv_heads, a.head_dim)
            v = a.v_proj(h).view(T, a.num_kv_heads, a.head_dim)
            mix = a.o_proj(cp_attention(q, k, v, self.cp.group, a.scaling).reshape(T, -1))
        else:
            mix = self.self_attn(h, pos, cos_t, sin_t, cu)
        x = torch.add(x, mix, alpha=rm)
        y = self.post_attention_layernorm(x)
        out = 0
        if self.block_sparse_moe is not None:
            moe = self.block_sparse_moe(y)
            out = moe[0] if isinstance(moe, tuple) else moe
        if self.shared_mlp is not None:
            out = out + self.shared_mlp(y)
        return torch.add(x, out, alpha=rm)


class GraniteMoeHybridModel(nn.Module):
    def __init__(self, cfg: DecoderConfig, layer_hook=None):
        super().__init__()
        self.cfg = cfg
        self.embed_tokens = nn.Embedding(cfg.vocab_size, cfg.hidden_size)
        nn.init.normal_(self.embed_tokens.weight, 0.0, cfg.initializer_range)
        layers = []
        for i in range(cfg.num_hidden_layers):
            layer = GraniteMoeHybridDecoderLayer(cfg, i)
            layer.apply(lambda m: _init_weights(m, cfg.initializer_range))
            if layer_hook is not None:
                layer = layer_hook(layer) or layer
            layers.append(layer)
        self.layers = nn.ModuleList(layers)
        self.norm = LlamaRMSNorm(cfg.hidden_size, cfg.rms_norm_eps)
        self.fused = False

    def forward(self, input_ids, position_ids=None, cu_seqlens=None, max_seqlen=None):
        B, S = input_ids.shape
        T = B * S
        dev = input_ids.device
        x = self.embed_tokens(input_ids.reshape(-1)) * self.cfg.embedding_multiplier
        if cu_seqlens is not None:
            cu = [int(c) for c in cu_seqlens.tolist()]
        elif position_ids is not None:
            cu = torch.nonzero(position_ids.reshape(-1) == 0).reshape(-1).tolist() + [T]
        else:
            cu = list(range(0, T + 1, S))
        # identity rotation: the attention layers of this family use no positional embedding
        cos_t = torch.ones(1, self.cfg.head_dim // 2, device=dev)
        sin_t = torch.zeros(1, self.cfg.head_dim // 2, device=dev)
        pos = torch.zeros(T, dtype=torch.long, device=dev)
        for layer in self.layers:
            x = _run_layer(self, layer, x, pos, cos_t, sin_t, cu)
        return self.norm(x)


class GraniteMoeHybridForCausalLM(LlamaForCausalLM):
    model_cls = GraniteMoeHybridModel
