"""Per-architecture descriptions: where the decoder layers live and in which order the linears inside one
layer are quantised (modules in the same inner list share calibration inputs).  Same information as the
per-family files of the reference (fms_acceleration_peft/gptqmodel/models/llama.py:20-38, mixtral.py:20-56,
gpt_bigcode.py, gpt_neox.py, granite.py:20-30, dbrx*.py)."""
from .base import BaseGPTQModel

_LLAMA_LAYER = [
    ["self_attn.k_proj", "self_attn.v_proj", "self_attn.q_proj"],
    ["self_attn.o_proj"],
    ["mlp.up_proj", "mlp.gate_proj"],
    ["mlp.down_proj"],
]


class LlamaGPTQ(BaseGPTQModel):
    base_modules = ["model.embed_tokens", "model.norm"]
    layers_node = "model.layers"
    layer_type = "LlamaDecoderLayer"
    layer_modules = _LLAMA_LAYER


class MistralGPTQ(LlamaGPTQ):
    layer_type = "MistralDecoderLayer"


class GemmaGPTQ(LlamaGPTQ):
    layer_type = "GemmaDecoderLayer"


class GraniteGPTQ(LlamaGPTQ):
    layer_type = "GraniteDecoderLayer"


class MixtralGPTQ(BaseGPTQModel):
    base_modules = ["model.embed_tokens", "model.norm"]
    layers_node = "model.layers"
    layer_type = "MixtralDecoderLayer"
    dynamic_expert_index = "num_local_experts"
    layer_modules = [
        ["self_attn.k_proj", "self_attn.v_proj", "self_attn.q_proj"],
        ["self_attn.o_proj"],
        ["block_sparse_moe.experts.{expert_index}.w1", "block_sparse_moe.experts.{expert_index}.w3"],
        ["block_sparse_moe.experts.{expert_index}.w2"],
    ]


class GPTBigCodeGPTQ(BaseGPTQModel):
    base_modules = ["transformer.wpe", "transformer.wte", "transformer.ln_f"]
    layers_node = "transformer.h"
    layer_type = "GPTBigCodeBlock"
    layer_modules = [["attn.c_attn"], ["attn.c_proj"], ["mlp.c_fc"], ["mlp.c_proj"]]


class GPTNeoXGPTQ(BaseGPTQModel):
    base_modules = ["gpt_neox.embed_in", "gpt_neox.final_layer_norm"]
    lm_head = "embed_out"
    layers_node = "gpt_neox.layers"
    layer_type = "GPTNeoXLayer"
    layer_modules = [["attention.query_key_value"], ["attention.dense"], ["mlp.dense_h_to_4h"], ["mlp.dense_4h_to_h"]]


class DbrxGPTQ(BaseGPTQModel):
    # the stock DBRX checkpoint stores fused expert tensors that cannot be packed: convert first
    info = {"notes": "DBRX must be converted to the per-expert linear layout before quantisation"}


class DbrxConvertedGPTQ(BaseGPTQModel):
    require_trust_remote_code = True  # the converted layout exists only as remote code on the Hugging Face side
    base_modules = ["transformer.wte", "transformer.norm_f"]
    layers_node = "transformer.blocks"
    layer_type = "DbrxBlock"
    dynamic_expert_index = "ffn_config.moe_num_experts"
    layer_modules = [
        ["norm_attn_norm.attn.q_proj", "norm_attn_norm.attn.k_proj", "norm_attn_norm.attn.v_proj"],
        ["norm_attn_norm.attn.out_proj"],
        ["ffn.experts.mlp.{expert_index}.w1", "ffn.experts.mlp.{expert_index}.v1"],
        ["ffn.experts.mlp.{expert_index}.w2"],
    ]
