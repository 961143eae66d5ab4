"""Every model family of the zoo builds, runs forward/backward on the CPU and keeps Hugging Face parameter names."""
import pytest
import torch

from fms_acceleration_b200.models.builder import build_model, resolve_config
from fms_acceleration_b200.models.config import HUB_ALIASES, PRESETS

TINY = ["tiny-llama", "tiny-granitemoe", "tiny-mixtral", "tiny-granitemoeshared", "tiny-gpt-bigcode",
        "tiny-granitemoehybrid", "tiny-mamba2"]


@pytest.mark.parametrize("name", TINY)
def test_forward_backward(name):
    torch.manual_seed(0)
    model = build_model(name, dtype=torch.float32, seed=0)
    V = model.config.vocab_size
    ids = torch.randint(0, V, (1, 48))
    kwargs = {} if "mamba2" in name else {"cu_seqlens": torch.tensor([0, 20, 48], dtype=torch.int32)}
    out = model(input_ids=ids, labels=ids.clone(), **kwargs)
    assert torch.isfinite(out.loss) and abs(float(out.loss) - torch.log(torch.tensor(float(V))).item()) < 1.5
    out.loss.backward()
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in model.parameters() if p.requires_grad)


@pytest.mark.parametrize("name", ["tiny-llama", "tiny-mixtral", "tiny-gpt-bigcode", "tiny-granitemoehybrid"])
def test_packed_documents_are_independent(name):
    """Logits of the second document do not depend on the tokens of the first."""
    torch.manual_seed(1)
    model = build_model(name, dtype=torch.float32, seed=1).eval()
    V = model.config.vocab_size
    a, b, b2 = torch.randint(0, V, (1, 16)), torch.randint(0, V, (1, 24)), torch.randint(0, V, (1, 16))
    cu = torch.tensor([0, 16, 40], dtype=torch.int32)
    with torch.no_grad():
        l1 = model(input_ids=torch.cat([a, b], 1), cu_seqlens=cu).logits[0, 16:]
        l2 = model(input_ids=torch.cat([b2, b], 1), cu_seqlens=cu).logits[0, 16:]
    assert torch.allclose(l1, l2, atol=1e-5)


def test_hf_parameter_names():
    names = {n for n, _ in build_model("tiny-mixtral").named_parameters()}
    assert "model.layers.0.block_sparse_moe.gate.weight" in names
    assert "model.layers.1.block_sparse_moe.experts.3.w2.weight" in names
    names = {n for n, _ in build_model("tiny-granitemoeshared").named_parameters()}
    assert "model.layers.0.shared_mlp.input_linear.weight" in names
    assert "model.layers.0.block_sparse_moe.input_linear.weight" in names
    names = {n for n, _ in build_model("tiny-gpt-bigcode").named_parameters()}
    assert {"transformer.wte.weight", "transformer.wpe.weight", "transformer.h.0.attn.c_attn.weight",
            "transformer.h.1.mlp.c_fc.bias", "transformer.ln_f.weight"} <= names
    names = {n for n, _ in build_model("tiny-granitemoehybrid").named_parameters()}
    assert "model.layers.0.mamba.in_proj.weight" in names and "model.layers.1.self_attn.q_proj.weight" in names


def test_hub_aliases_resolve_to_presets():
    for hub, name in HUB_ALIASES.items():
        assert name in PRESETS
        cfg = resolve_config(hub)
        assert cfg.architectures == PRESETS[name]().architectures
    assert resolve_config("mistralai/Mixtral-8x7B-Instruct-v0.1").num_local_experts == 8
