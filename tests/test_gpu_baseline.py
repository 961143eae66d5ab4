"""The library-kernel comparison arm on a GPU (cuBLAS, flash-attn, the reference's Triton kernels by path) computes
the same loss and gradients as the product path of the same model."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from fms_acceleration_b200 import _native as NV
from fms_acceleration_b200.baseline import BaselineRunner, reference_kernels_status
from fms_acceleration_b200.models.builder import build_model, quantize_linears_
from fms_acceleration_b200.models.config import DecoderConfig
from fms_acceleration_b200.nn import Linear4bit, LoraConfig, get_peft_model
from fms_acceleration_b200.trainer import synthetic_packed_batch, to_device

DEV = "cuda"


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp(min=1e-12)).item()


def test_qlora_decoder_product_vs_library_arm():
    cfg = DecoderConfig(vocab_size=4096, hidden_size=512, intermediate_size=1024, num_hidden_layers=2,
                        num_attention_heads=4, num_key_value_heads=2, head_dim=128, rope_theta=1e6,
                        architectures=["MistralForCausalLM"], model_type="mistral")
    model = build_model(cfg, device=DEV, dtype=torch.bfloat16, seed=0, layer_hook=lambda layer: quantize_linears_(
        layer, lambda lin: Linear4bit.from_linear(lin, "nf4", 64, torch.bfloat16)))
    model = get_peft_model(model, LoraConfig(r=16, lora_alpha=16, target_modules=["q_proj", "k_proj", "v_proj", "o_proj"]))
    torch.manual_seed(1)
    for n, p in model.named_parameters():
        if "lora_B" in n:
            torch.nn.init.normal_(p, std=0.02)
    model.get_base_model().enable_fused("fused_ce_liger")
    b = to_device(synthetic_packed_batch(4096, 2, 512, (32, 512), seed=0, pin=False), DEV)
    kw = dict(input_ids=b["input_ids"], labels=b["labels"], cu_seqlens=b["cu_seqlens"])
    loss = model(**kw).loss
    loss.backward()
    NV.check_status()
    want = {n: p.grad.float().clone() for n, p in model.named_parameters() if p.grad is not None}
    model.zero_grad()
    runner = BaselineRunner(model)
    got = runner(**kw).loss
    got.backward()
    assert abs(got.item() - loss.item()) < 3e-2
    for n, p in model.named_parameters():
        if n in want and want[n].norm() > 1e-6:
            assert _rel(p.grad, want[n]) < 8e-2, n
    st = reference_kernels_status()
    assert "flash_attn" in st["attention"]


def test_moe_decoder_product_vs_library_arm():
    from fms_acceleration_b200.plugins.moe.utils import prepare_scattermoe

    model = build_model("tiny-granitemoe", device=DEV, dtype=torch.bfloat16, seed=0)
    prepare_scattermoe(model, None, 0, 1, 1)
    model.enable_fused("fused_ce_liger")
    b = to_device(synthetic_packed_batch(1024, 2, 256, (16, 256), seed=5, pin=False), DEV)
    kw = dict(input_ids=b["input_ids"], labels=b["labels"], cu_seqlens=b["cu_seqlens"])
    loss = model(**kw).loss
    runner = BaselineRunner(model)
    got = runner(**kw).loss
    got.backward()
    NV.check_status()
    assert abs(got.item() - loss.item()) < 5e-2, (got.item(), loss.item(), reference_kernels_status())
    assert all(torch.isfinite(p.grad).all() for p in model.parameters() if p.grad is not None)
