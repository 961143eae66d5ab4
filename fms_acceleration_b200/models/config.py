"""Architecture descriptions for the in-tree model zoo and the presets used by the benchmarks."""
from __future__ import annotations

from dataclasses import dataclass, field, asdict
from typing import List, Optional


@dataclass
class DecoderConfig:
    vocab_size: int = 32000
    hidden_size: int = 4096
    intermediate_size: int = 11008
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: Optional[int] = None
    head_dim: Optional[int] = None
    hidden_act: str = "silu"
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    max_position_embeddings: int = 4096
    tie_word_embeddings: bool = False
    initializer_range: float = 0.02
    model_type: str = "llama"
    architectures: List[str] = field(default_factory=lambda: ["LlamaForCausalLM"])
    # granite-style scalars
    embedding_multiplier: float = 1.0
    attention_multiplier: Optional[float] = None
    residual_multiplier: float = 1.0
    logits_scaling: float = 1.0
    # mixture of experts
    num_local_experts: int = 0
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0
    shared_intermediate_size: int = 0
    router_aux_loss_coef: float = 0.0
    # mamba2
    mamba_d_state: int = 128
    mamba_d_conv: int = 4
    mamba_expand: int = 2
    mamba_d_head: int = 64
    mamba_n_groups: int = 1
    mamba_chunk_size: int = 256
    mamba_conv_bias: bool = True
    mamba_proj_bias: bool = False
    # hybrid decoders: "mamba" or "attention" per layer (empty: the family's default)
    layer_types: List[str] = field(default_factory=list)
    name_or_path: str = ""
    torch_dtype: str = "bfloat16"

    def __post_init__(self):
        if self.num_key_value_heads is None:
            self.num_key_value_heads = self.num_attention_heads
        if self.head_dim is None:
            self.head_dim = self.hidden_size // self.num_attention_heads

    def to_dict(self):
        return asdict(self)


def tiny_llama() -> DecoderConfig:
    """2-layer Llama used for CPU plumbing tests."""
    return DecoderConfig(vocab_size=32000, hidden_size=256, intermediate_size=688, num_hidden_layers=2,
                         num_attention_heads=4, num_key_value_heads=4, rms_norm_eps=1e-6, rope_theta=10000.0,
                         max_position_embeddings=2048)


def mistral_7b() -> DecoderConfig:
    return DecoderConfig(vocab_size=32000, hidden_size=4096, intermediate_size=14336, num_hidden_layers=32,
                         num_attention_heads=32, num_key_value_heads=8, rms_norm_eps=1e-5, rope_theta=1e6,
                         max_position_embeddings=32768, model_type="mistral", architectures=["MistralForCausalLM"])


def llama2_70b() -> DecoderConfig:
    return DecoderConfig(vocab_size=32000, hidden_size=8192, intermediate_size=28672, num_hidden_layers=80,
                         num_attention_heads=64, num_key_value_heads=8, rms_norm_eps=1e-5, rope_theta=10000.0,
                         max_position_embeddings=4096, model_type="llama", architectures=["LlamaForCausalLM"])


def granite_3b_a800m() -> DecoderConfig:
    return DecoderConfig(vocab_size=49155, hidden_size=1536, intermediate_size=512, num_hidden_layers=32,
                         num_attention_heads=24, num_key_value_heads=8, rms_norm_eps=1e-6, rope_theta=10000.0,
                         max_position_embeddings=4096, tie_word_embeddings=True, model_type="granitemoe",
                         architectures=["GraniteMoeForCausalLM"], num_local_experts=40, num_experts_per_tok=8,
                         moe_intermediate_size=512)


def tiny_granitemoe() -> DecoderConfig:
    return DecoderConfig(vocab_size=1024, hidden_size=256, intermediate_size=128, num_hidden_layers=2,
                         num_attention_heads=4, num_key_value_heads=2, tie_word_embeddings=True,
                         model_type="granitemoe", architectures=["GraniteMoeForCausalLM"], num_local_experts=8,
                         num_experts_per_tok=2, moe_intermediate_size=128)


def mamba2_2p7b() -> DecoderConfig:
    return DecoderConfig(vocab_size=50288, hidden_size=2560, num_hidden_layers=64, num_attention_heads=80,
                         model_type="mamba2", architectures=["Mamba2ForCausalLM"], mamba_d_state=128,
                         mamba_d_head=64, mamba_expand=2, mamba_d_conv=4, mamba_chunk_size=256, rms_norm_eps=1e-5,
                         tie_word_embeddings=True)


def tiny_mamba2() -> DecoderConfig:
    return DecoderConfig(vocab_size=512, hidden_size=128, num_hidden_layers=2, num_attention_heads=4,
                         model_type="mamba2", architectures=["Mamba2ForCausalLM"], mamba_d_state=32, mamba_d_head=32,
                         mamba_expand=2, mamba_d_conv=4, mamba_chunk_size=32, rms_norm_eps=1e-5,
                         tie_word_embeddings=True)


def mixtral_8x7b() -> DecoderConfig:
    return DecoderConfig(vocab_size=32000, hidden_size=4096, intermediate_size=14336, num_hidden_layers=32,
                         num_attention_heads=32, num_key_value_heads=8, rms_norm_eps=1e-5, rope_theta=1e6,
                         max_position_embeddings=32768, model_type="mixtral", architectures=["MixtralForCausalLM"],
                         num_local_experts=8, num_experts_per_tok=2, moe_intermediate_size=14336)


def tiny_mixtral() -> DecoderConfig:
    return DecoderConfig(vocab_size=1024, hidden_size=256, intermediate_size=128, num_hidden_layers=2,
                         num_attention_heads=4, num_key_value_heads=2, model_type="mixtral",
                         architectures=["MixtralForCausalLM"], num_local_experts=4, num_experts_per_tok=2,
                         moe_intermediate_size=128)


def granite_8b() -> DecoderConfig:
    """Granite 3 dense 8B."""
    return DecoderConfig(vocab_size=49155, hidden_size=4096, intermediate_size=12800, num_hidden_layers=40,
                         num_attention_heads=32, num_key_value_heads=8, rms_norm_eps=1e-5, rope_theta=10000.0,
                         max_position_embeddings=4096, tie_word_embeddings=True, model_type="granite",
                         architectures=["GraniteForCausalLM"], embedding_multiplier=12.0, attention_multiplier=0.0078125,
                         residual_multiplier=0.22, logits_scaling=16.0)


def tiny_granitemoeshared() -> DecoderConfig:
    return DecoderConfig(vocab_size=1024, hidden_size=256, intermediate_size=128, num_hidden_layers=2,
                         num_attention_heads=4, num_key_value_heads=2, tie_word_embeddings=True,
                         model_type="granitemoeshared", architectures=["GraniteMoeSharedForCausalLM"],
                         num_local_experts=8, num_experts_per_tok=2, moe_intermediate_size=128,
                         shared_intermediate_size=192)


def santacoder() -> DecoderConfig:
    """bigcode/gpt_bigcode-santacoder: multi-query attention, learned positions, GELU MLP."""
    return DecoderConfig(vocab_size=49280, hidden_size=2048, intermediate_size=8192, num_hidden_layers=24,
                         num_attention_heads=16, num_key_value_heads=1, rms_norm_eps=1e-5, max_position_embeddings=2048,
                         tie_word_embeddings=True, hidden_act="gelu_pytorch_tanh", model_type="gpt_bigcode",
                         architectures=["GPTBigCodeForCausalLM"])


def tiny_gpt_bigcode() -> DecoderConfig:
    return DecoderConfig(vocab_size=1024, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                         num_attention_heads=4, num_key_value_heads=1, rms_norm_eps=1e-5, max_position_embeddings=512,
                         tie_word_embeddings=True, hidden_act="gelu_pytorch_tanh", model_type="gpt_bigcode",
                         architectures=["GPTBigCodeForCausalLM"])


def tiny_granitemoehybrid() -> DecoderConfig:
    return DecoderConfig(vocab_size=512, hidden_size=128, intermediate_size=64, num_hidden_layers=4,
                         num_attention_heads=4, num_key_value_heads=2, tie_word_embeddings=True,
                         model_type="granitemoehybrid", architectures=["GraniteMoeHybridForCausalLM"],
                         num_local_experts=4, num_experts_per_tok=2, moe_intermediate_size=64,
                         shared_intermediate_size=96, mamba_d_state=32, mamba_d_head=32, mamba_chunk_size=32,
                         layer_types=["mamba", "attention", "mamba", "mamba"])


# The presets below take their shapes from the model cards as remembered (there is no network here to fetch the
# configuration files); weights are random-init, so only the shapes matter for the benchmark scenarios that name them.
def llama3_8b() -> DecoderConfig:
    return DecoderConfig(vocab_size=128256, hidden_size=4096, intermediate_size=14336, num_hidden_layers=32,
                         num_attention_heads=32, num_key_value_heads=8, rms_norm_eps=1e-5, rope_theta=500000.0,
                         max_position_embeddings=8192, model_type="llama", architectures=["LlamaForCausalLM"])


def powerlm_3b() -> DecoderConfig:
    """ibm/PowerLM-3b: dense Granite-architecture decoder."""
    return DecoderConfig(vocab_size=49152, hidden_size=2304, intermediate_size=9216, num_hidden_layers=40,
                         num_attention_heads=36, num_key_value_heads=36, rms_norm_eps=1e-5, rope_theta=10000.0,
                         max_position_embeddings=4096, tie_word_embeddings=True, model_type="granite",
                         architectures=["GraniteForCausalLM"], embedding_multiplier=12.0, attention_multiplier=0.015625,
                         residual_multiplier=0.22, logits_scaling=8.0)


def powermoe_3b() -> DecoderConfig:
    """ibm/PowerMoE-3b: 40 experts, 8 active (the shapes of granite-3.0-3b-a800m)."""
    return DecoderConfig(vocab_size=49152, hidden_size=1536, intermediate_size=512, num_hidden_layers=32,
                         num_attention_heads=24, num_key_value_heads=8, rms_norm_eps=1e-6, rope_theta=10000.0,
                         max_position_embeddings=4096, tie_word_embeddings=True, model_type="granitemoe",
                         architectures=["GraniteMoeForCausalLM"], num_local_experts=40, num_experts_per_tok=8,
                         moe_intermediate_size=512, embedding_multiplier=12.0, attention_multiplier=0.015625,
                         residual_multiplier=0.22, logits_scaling=6.0)


def granite_moe_7b_1b_shared() -> DecoderConfig:
    """ibm-research/moe-7b-1b-active-shared-experts: 62 routed experts, 6 active, plus a shared dense branch."""
    return DecoderConfig(vocab_size=49160, hidden_size=1536, intermediate_size=512, num_hidden_layers=40,
                         num_attention_heads=12, num_key_value_heads=4, rms_norm_eps=1e-5, rope_theta=10000.0,
                         max_position_embeddings=8192, tie_word_embeddings=True, model_type="granitemoeshared",
                         architectures=["GraniteMoeSharedForCausalLM"], num_local_experts=62, num_experts_per_tok=6,
                         moe_intermediate_size=512, shared_intermediate_size=1024, embedding_multiplier=12.0,
                         attention_multiplier=0.0078125, residual_multiplier=0.22, logits_scaling=6.0)


def granite_4_tiny_preview() -> DecoderConfig:
    """ibm-granite/granite-4.0-tiny-preview: the same feed-forward, Mamba2 mixers with an attention layer every tenth
    layer (5, 15, 25, 35), no positional embedding."""
    cfg = granite_moe_7b_1b_shared()
    cfg.model_type, cfg.architectures = "granitemoehybrid", ["GraniteMoeHybridForCausalLM"]
    cfg.mamba_d_state, cfg.mamba_d_head, cfg.mamba_expand, cfg.mamba_d_conv = 128, 64, 2, 4
    cfg.mamba_n_groups, cfg.mamba_chunk_size = 1, 256
    cfg.layer_types = ["attention" if i % 10 == 5 else "mamba" for i in range(cfg.num_hidden_layers)]
    return cfg


PRESETS = {
    "tiny-llama": tiny_llama,
    "mistral-7b": mistral_7b,
    "llama2-70b": llama2_70b,
    "granite-3b-a800m": granite_3b_a800m,
    "tiny-granitemoe": tiny_granitemoe,
    "mamba2-2.7b": mamba2_2p7b,
    "tiny-mamba2": tiny_mamba2,
    "mixtral-8x7b": mixtral_8x7b,
    "tiny-mixtral": tiny_mixtral,
    "granite-8b": granite_8b,
    "tiny-granitemoeshared": tiny_granitemoeshared,
    "santacoder": santacoder,
    "tiny-gpt-bigcode": tiny_gpt_bigcode,
    "tiny-granitemoehybrid": tiny_granitemoehybrid,
    "llama3-8b": llama3_8b,
    "powerlm-3b": powerlm_3b,
    "powermoe-3b": powermoe_3b,
    "granite-moe-7b-1b-shared": granite_moe_7b_1b_shared,
    "granite-4.0-tiny-preview": granite_4_tiny_preview,
}

# Hugging Face hub ids used by the reference's benchmark scenarios -> the preset of the same architecture
# (weights are random-init here; only the shapes are taken from the named model).
HUB_ALIASES = {
    "mistralai/Mistral-7B-v0.1": "mistral-7b",
    "TheBloke/Mistral-7B-v0.1-GPTQ": "mistral-7b",
    "NousResearch/Llama-2-70b-hf": "llama2-70b",
    "TheBloke/Llama-2-70B-GPTQ": "llama2-70b",
    "mistralai/Mixtral-8x7B-Instruct-v0.1": "mixtral-8x7b",
    "TheBloke/Mixtral-8x7B-Instruct-v0.1-GPTQ": "mixtral-8x7b",
    "ibm-granite/granite-3.0-3b-a800m-instruct": "granite-3b-a800m",
    "ibm-granite/granite-3.0-8b-instruct": "granite-8b",
    "bigcode/gpt_bigcode-santacoder": "santacoder",
    "state-spaces/mamba2-2.7b": "mamba2-2.7b",
    "meta-llama/Meta-Llama-3-8B": "llama3-8b",
    "TechxGenus/Meta-Llama-3-8B-GPTQ": "llama3-8b",
    "ibm/PowerLM-3b": "powerlm-3b",
    "ibm/PowerMoE-3b": "powermoe-3b",
    "ibm-research/moe-7b-1b-active-shared-experts": "granite-moe-7b-1b-shared",
    "ibm-granite/granite-4.0-tiny-preview": "granite-4.0-tiny-preview",
}


def preset(name: str) -> DecoderConfig:
    return PRESETS[HUB_ALIASES.get(name, name)]()
