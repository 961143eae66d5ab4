"""Mamba2 language model with Hugging Face / mamba_ssm parameter names (``in_proj``, ``conv1d``, ``dt_bias``, ``A_log``,
``D``, ``norm``, ``out_proj``), the parameter set the reference's context-parallel swap relies on
(fms_acceleration_mcp/utils/utils.py:87-140).

Block: ``zxbcdt = in_proj(u)``; split into gate ``z``, conv input ``xBC`` and ``dt``; depthwise causal conv (kernel
``d_conv``) + SiLU over ``xBC``; split into ``x, B, C``; ``dt = softplus(dt + dt_bias)``; SSD scan with
``A = -exp(A_log)`` and skip ``D``; gated RMSNorm ``norm(y * silu(z))``; ``out_proj``.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F
from torch import nn

from ..ops import activation as ACT
from ..ops import cross_entropy as CE
from ..ops import mamba as MB
from ..ops import rmsnorm as RN
from .config import DecoderConfig
from .generation import GenerationMixin
from .llama import CausalLMOutput, LlamaRMSNorm, _DenseLinear, _init_weights, _run_layer


class MambaRMSNormGated(nn.Module):
    def __init__(self, hidden_size: int, eps: float = 1e-5):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden_size))
        self.variance_epsilon = eps

    def forward(self, y, z):
        if y.is_cuda and y.dtype in (torch.bfloat16, torch.float16):
            return RN.rmsnorm(ACT.glu(z, y, "silu"), self.weight, self.variance_epsilon)
        h = (y.float() * F.silu(z.float())).to(y.dtype)
        out, _ = RN.rmsnorm_ref(h, self.weight, self.variance_epsilon)
        return out


def _aligned(t: torch.Tensor) -> torch.Tensor:
    """Row-contiguous view with 16-byte aligned rows (what the kernels' vector accesses need), copying if not."""
    if t.stride(-1) == 1 and t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0:
        return t
    return t.contiguous()


class _SplitCols(torch.autograd.Function):
    """Column blocks of a 2-D tensor as views.  The backward is ONE concatenation of the block gradients; the
    stock slicing backward zero-fills a full-width tensor per block and then adds them up."""

    @staticmethod
    def forward(ctx, t, *sizes):
        ctx.sizes, ctx.rows, ctx.meta = sizes, t.shape[0], (t.dtype, t.device)
        return tuple(t.split(list(sizes), dim=1))

    @staticmethod
    def backward(ctx, *grads):
        dtype, dev = ctx.meta
        parts = [g if g is not None else torch.zeros(ctx.rows, n, dtype=dtype, device=dev)
                 for g, n in zip(grads, ctx.sizes)]
        return (torch.cat(parts, dim=1),) + (None,) * len(ctx.sizes)


def _linear(x, lin: nn.Linear):
    if (x.is_cuda and x.dtype in (torch.bfloat16, torch.float16) and lin.bias is None
            and lin.in_features % 8 == 0 and lin.out_features % 8 == 0):
        return _DenseLinear.apply(x, lin.weight)
    return lin(x)


class Mamba2Mixer(nn.Module):
    def __init__(self, cfg: DecoderConfig, layer_idx: int):
        super().__init__()
        self.cfg = cfg
        self.layer_idx = layer_idx
        self.d_model = cfg.hidden_size
        self.d_inner = cfg.mamba_expand * cfg.hidden_size
        self.headdim = cfg.mamba_d_head
        self.nheads = self.d_inner // self.headdim
        self.d_state, self.ngroups, self.d_conv = cfg.mamba_d_state, cfg.mamba_n_groups, cfg.mamba_d_conv
        self.chunk_size = cfg.mamba_chunk_size
        self.conv_dim = self.d_inner + 2 * self.ngroups * self.d_state
        d_in_proj = 2 * self.d_inner + 2 * self.ngroups * self.d_state + self.nheads
        self.in_proj = nn.Linear(self.d_model, d_in_proj, bias=cfg.mamba_proj_bias)
        self.conv1d = nn.Conv1d(self.conv_dim, self.conv_dim, kernel_size=self.d_conv, groups=self.conv_dim,
                                padding=self.d_conv - 1, bias=cfg.mamba_conv_bias)
        dt = torch.exp(torch.rand(self.nheads) * (math.log(1e-1) - math.log(1e-3)) + math.log(1e-3)).clamp(min=1e-4)
        self.dt_bias = nn.Parameter(dt + torch.log(-torch.expm1(-dt)))  # inverse softplus
        self.A_log = nn.Parameter(torch.log(torch.empty(self.nheads).uniform_(1, 16)))
        self.D = nn.Parameter(torch.ones(self.nheads))
        self.norm = MambaRMSNormGated(self.d_inner, cfg.rms_norm_eps)
        self.out_proj = nn.Linear(self.d_inner, self.d_model, bias=cfg.mamba_proj_bias)
        # context parallelism (installed by the mamba-cp plugin)
        self.cp = None

    def forward(self, u: torch.Tensor, seq_start=None, seq_end=None) -> torch.Tensor:
        """u: [T, d_model] packed tokens of one (slice of a) sequence."""
        T = u.shape[0]
        zxbcdt = _linear(u, self.in_proj)
        di, gn = self.d_inner, self.ngroups * self.d_state
        z, xBC, dt_raw = _SplitCols.apply(zxbcdt, di, self.conv_dim, zxbcdt.shape[1] - di - self.conv_dim)
        w = self.conv1d.weight.squeeze(1)
        halo = self.cp.exchange_halo(xBC, self.d_conv - 1, self.layer_idx) if self.cp is not None else None
        xs, BC = MB.causal_conv1d(_aligned(xBC), w.to(xBC.dtype),
                                  None if self.conv1d.bias is None else self.conv1d.bias.to(xBC.dtype), halo, seq_start,
                                  seq_end, split=di)
        Bs, Cs = _SplitCols.apply(BC, gn, gn)
        x = xs.reshape(T, self.nheads, self.headdim)
        B = Bs.reshape(T, self.ngroups, self.d_state)
        C = Cs.reshape(T, self.ngroups, self.d_state)
        dt = F.softplus(dt_raw.float() + self.dt_bias.float())
        A = -torch.exp(self.A_log.float())
        Q = min(self.chunk_size, T)
        pad = (-T) % Q
        if pad:
            x, B, C = (F.pad(t, (0, 0, 0, 0, 0, pad)) for t in (x, B, C))
            dt = F.pad(dt, (0, 0, 0, pad))
        if self.cp is not None:
            y = self.cp.scan(x.contiguous(), dt, A, B.contiguous(), C.contiguous(), self.D.float(), Q, self.layer_idx)
        else:
            y, _ = MB.ssd_scan(x.contiguous(), dt, A, B.contiguous(), C.contiguous(), self.D.float(), None, Q)
        if pad:  # an unconditional y[:T] records a slice whose backward zero-fills and copies a [T, d_inner] tensor
            y = y[:T]
        y = y.reshape(T, di)
        y = self.norm(_aligned(y), _aligned(z))
        return _linear(y, self.out_proj)


class Mamba2Block(nn.Module):
    def __init__(self, cfg: DecoderConfig, layer_idx: int):
        super().__init__()
        self.norm = LlamaRMSNorm(cfg.hidden_size, cfg.rms_norm_eps)
        self.mamba = Mamba2Mixer(cfg, layer_idx)  # attribute name used by the context-parallel swap
        self.mixer = self.mamba

    def forward(self, x):
        h = RN.rmsnorm(x, self.norm.weight, self.norm.variance_epsilon) if x.is_cuda else self.norm(x)
        return x + self.mamba(h)


class Mamba2Model(nn.Module):
    def __init__(self, cfg: DecoderConfig, layer_hook=None):
        super().__init__()
        self.cfg = cfg
        self.embed_tokens = nn.Embedding(cfg.vocab_size, cfg.hidden_size)
        nn.init.normal_(self.embed_tokens.weight, 0.0, cfg.initializer_range)
        layers = []
        for i in range(cfg.num_hidden_layers):
            blk = Mamba2Block(cfg, i)
            blk.apply(lambda m: _init_weights(m, cfg.initializer_range))
            if layer_hook is not None:
                blk = layer_hook(blk) or blk
            layers.append(blk)
        self.layers = nn.ModuleList(layers)
        self.norm_f = LlamaRMSNorm(cfg.hidden_size, cfg.rms_norm_eps)
        self.fused = False

    def forward(self, input_ids):
        x = self.embed_tokens(input_ids.reshape(-1))
        for blk in self.layers:
            x = _run_layer(self, blk, x)
        return RN.rmsnorm(x, self.norm_f.weight, self.norm_f.variance_epsilon) if x.is_cuda else self.norm_f(x)


class Mamba2ForCausalLM(GenerationMixin, nn.Module):
    def __init__(self, cfg: DecoderConfig, layer_hook=None):
        super().__init__()
        self.config = cfg
        self.model = Mamba2Model(cfg, layer_hook)
        self.backbone = self.model
        self.lm_head = nn.Linear(cfg.hidden_size, cfg.vocab_size, bias=False)
        if cfg.tie_word_embeddings:
            self.lm_head.weight = self.model.embed_tokens.weight
        else:
            nn.init.normal_(self.lm_head.weight, 0.0, cfg.initializer_range)
        self.fast_loss = False
        self.cp = None  # context-parallel state (set by the plugin): shifts labels across rank boundaries

    def enable_fused(self, fast_loss="fused_ce_liger"):
        self.fast_loss = fast_loss
        return self

    def gradient_checkpointing_enable(self, gradient_checkpointing_kwargs=None, **kwargs):
        self.model.gradient_checkpointing = True

    def gradient_checkpointing_disable(self):
        self.model.gradient_checkpointing = False

    def forward(self, input_ids, labels=None, num_items_in_batch=None, **kwargs):
        """One sequence (or this rank's slice of it under context parallelism): ``input_ids [1, T]``."""
        hidden = self.model(input_ids)
        loss = logits = None
        if labels is not None:
            flat = labels.reshape(-1)
            if self.cp is not None:
                shift = self.cp.shift_labels(flat)
            else:
                shift = torch.cat([flat[1:], flat.new_full((1,), CE.IGNORE_INDEX)])
            if hidden.is_cuda and self.fast_loss == "fused_ce_liger":
                if self.cp is not None:
                    # mean over the tokens of ALL ranks: sum locally, divide by the global count
                    n = self.cp.global_count(shift != CE.IGNORE_INDEX)
                    loss = CE.fused_linear_cross_entropy(hidden, self.lm_head.weight, shift, num_items=n)
                else:
                    loss = CE.fused_linear_cross_entropy(hidden, self.lm_head.weight, shift, num_items=num_items_in_batch)
            else:
                logits = self.lm_head(hidden)
                per = CE.cross_entropy_ref(logits, shift) if not (self.fast_loss and logits.is_cuda) else \
                    CE.fast_cross_entropy_loss(logits, shift)
                if num_items_in_batch is not None:
                    n = num_items_in_batch
                elif self.cp is not None:
                    n = self.cp.global_count(shift != CE.IGNORE_INDEX).reshape(())  # tokens of ALL ranks, as above
                else:
                    n = (shift != CE.IGNORE_INDEX).sum().clamp(min=1)
                loss = per.sum() / n
        else:
            logits = self.lm_head(hidden)
        return CausalLMOutput(loss=loss, logits=None if logits is None else logits.view(*input_ids.shape, -1))
