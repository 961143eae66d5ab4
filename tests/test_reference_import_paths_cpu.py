"""Module paths of the reference's packages that user code may import (kernels, fused ops, per-family rule modules,
the GPTQ layer) resolve under the alias packages to the in-tree implementations, and the pieces that have a CPU
oracle path compute the right thing."""
import importlib

import pytest
import torch

PATHS = [
    "fms_acceleration_foak.kernels.unsloth.rms_layernorm", "fms_acceleration_foak.kernels.unsloth.rope_embedding",
    "fms_acceleration_foak.kernels.unsloth.cross_entropy_loss", "fms_acceleration_foak.kernels.unsloth.utils",
    "fms_acceleration_foak.fused_ops.liger_ce.cross_entropy",
    "fms_acceleration_foak.fused_ops.liger_ce.fused_linear_cross_entropy_loss",
    "fms_acceleration_foak.fused_ops.unsloth_lora.swiglu", "fms_acceleration_foak.fused_ops.unsloth_lora.geglu",
    "fms_acceleration_foak.fused_ops.unsloth_lora.utils", "fms_acceleration_foak.fused_ops.unsloth_lora.bnb.fast_lora",
    "fms_acceleration_foak.fused_ops.unsloth_lora.gptq.fast_lora",
    "fms_acceleration_foak.fused_ops.unsloth_lora.gptq.triton.kernels",
    "fms_acceleration_foak.models.llama", "fms_acceleration_foak.models.mistral", "fms_acceleration_foak.models.granite",
    "fms_acceleration_foak.models.mixtral", "fms_acceleration_foak.models.granitemoe",
    "fms_acceleration_foak.models.granitemoeshared", "fms_acceleration_foak.models.granitemoehybrid",
    "fms_acceleration_foak.models.gpt_bigcode", "fms_acceleration_foak.models.utils",
    "fms_acceleration_peft.gptqmodel.nn_modules.qlinear.qlinear_tritonv2",
    "fms_acceleration_peft.gptqmodel.utils.importer", "fms_acceleration_moe.utils.scattermoe_state_dict",
    "fms_acceleration_aadp.multipack_sampler", "fms_acceleration_odm.odm.dataset", "fms_acceleration_mcp.utils.utils",
    "fms_acceleration.utils.test_utils",
]


@pytest.mark.parametrize("path", PATHS)
def test_reference_module_path_resolves(path):
    mod = importlib.import_module(path)
    # the alias gives the module object of the implementation, not a second copy
    assert mod.__name__.startswith("fms_acceleration_b200.")
    assert importlib.import_module(mod.__name__) is mod


def test_rule_modules_give_the_family_rules():
    from fms_acceleration_foak.models.gpt_bigcode import get_mp_rules as bigcode
    from fms_acceleration_foak.models.llama import get_mp_rules as llama

    ids = {r.rule_id for r in llama("bitsandbytes")}
    assert {"llama-rms", "llama-qkvo", "llama-mlp", "llama-rope", "llama-fused-lce"} <= ids
    assert all(r.rule_id.startswith("gpt_bigcode-") for r in bigcode("auto_gptq"))


def test_lora_matmul_and_losses_on_the_cpu():
    from fms_acceleration_foak.fused_ops.liger_ce.fused_linear_cross_entropy_loss import LigerFusedLinearCrossEntropyLoss
    from fms_acceleration_foak.fused_ops.unsloth_lora.utils import matmul_lora
    from fms_acceleration_foak.kernels.unsloth.cross_entropy_loss import FastForCausalLMLoss

    torch.manual_seed(0)
    X, W = torch.randn(2, 5, 8), torch.randn(6, 8)
    A, B = torch.randn(3, 8), torch.randn(6, 3)
    y = matmul_lora(X, W, None, A, B, 0.5)
    assert torch.allclose(y, X @ W.t() + 0.5 * (X @ A.t()) @ B.t(), atol=1e-5)
    logits, labels = torch.randn(2, 7, 11), torch.randint(0, 11, (2, 7))
    want = torch.nn.functional.cross_entropy(logits[:, :-1].reshape(-1, 11), labels[:, 1:].reshape(-1))
    assert torch.allclose(FastForCausalLMLoss(logits, labels), want, atol=1e-5)
    hidden, weight, target = torch.randn(9, 8), torch.randn(11, 8), torch.randint(0, 11, (9,))
    target[2] = -100
    got = LigerFusedLinearCrossEntropyLoss()(weight, hidden, target)
    assert torch.allclose(got, torch.nn.functional.cross_entropy(hidden @ weight.t(), target), atol=1e-5)


def test_gptq_state_helpers_on_the_cpu():
    from fms_acceleration_foak.fused_ops.unsloth_lora.gptq.fast_lora import dequantize, extract_gptq_state, unpack_gptqstate
    from fms_acceleration_foak.fused_ops.unsloth_lora.gptq.triton.kernels import dequant_ref
    from fms_acceleration_peft.gptqmodel.nn_modules.qlinear.qlinear_tritonv2 import QuantLinear

    layer = QuantLinear(4, 32, 64, 48, dtype=torch.float32)
    layer.qweight.random_(0, 2 ** 31 - 1)
    layer.qzeros.random_(0, 2 ** 31 - 1)
    layer.scales.uniform_(0.01, 0.02)
    st = extract_gptq_state(layer)
    assert len(unpack_gptqstate(st)) == 5 and st.bits == 4
    assert torch.equal(dequantize(st), dequant_ref(st)) and dequantize(st).shape == (64, 48)
