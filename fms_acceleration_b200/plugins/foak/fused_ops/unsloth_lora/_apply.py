"""The ``apply_lora_*`` entry points shared by the ``bnb`` and ``gptq`` flavours: ``self`` is an attention or MLP
module whose projections are LoRA-wrapped; the projections run as one projection group (one tcgen05 GEMM over the
concatenated base weight with the LoRA update accumulated in the same accumulator)."""
import torch

from fms_acceleration_b200.ops.activation import glu
from fms_acceleration_b200.ops.proj import ProjGroup
from fms_acceleration_b200.plugins.foak.models.utils import _GroupFn, _run_group

LoRA_QKV = LoRA_W = _GroupFn  # one autograd function serves every projection group


def _group(owner, names, tag):
    cache = owner.__dict__.setdefault("_fmsb_groups", {})
    g = cache.get(tag)
    if g is None:
        g = cache[tag] = ProjGroup([getattr(owner, n) for n in names], tag)
    return g


def apply_lora_qkv(self, X):
    """``(Q, K, V)`` of ``self.q_proj / k_proj / v_proj`` from one fused call."""
    g = _group(self, ["q_proj", "k_proj", "v_proj"], "qkv")
    y = _run_group(g, X)
    return tuple(torch.split(y, g.out_sizes, dim=-1))


def apply_lora_o(self, X):
    return _run_group(_group(self, ["o_proj"], "o"), X)


apply_lora_o_v2 = apply_lora_o


def _mlp(self, X, act):
    gu = _run_group(_group(self, ["gate_proj", "up_proj"], "gate_up"), X)
    e, g = torch.split(gu, gu.shape[-1] // 2, dim=-1)
    h = glu(e.reshape(-1, e.shape[-1]), g.reshape(-1, g.shape[-1]), act).view(*X.shape[:-1], e.shape[-1])
    return _run_group(_group(self, ["down_proj"], "down"), h)


def apply_lora_mlp_swiglu(self, X):
    return _mlp(self, X, "silu")


def apply_lora_mlp_geglu_exact(self, X):
    return _mlp(self, X, "gelu")


def apply_lora_mlp_geglu_approx(self, X):
    return _mlp(self, X, "gelu_pytorch_tanh")


apply_lora_mlp = apply_lora_mlp_swiglu


class LoRA_MLP:
    """The reference's single autograd function for the whole gated MLP; here the MLP is three projection groups
    and the activation kernel, each with its own backward."""

    @staticmethod
    def apply(X, mlp, act: str = "silu"):
        return _mlp(mlp, X, act)
