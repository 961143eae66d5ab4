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


def test_checkpoint_directories_load_plain_quantised_at_load_and_sharded(tmp_path):
    """``build_model`` on a directory with safetensors files: the plain model gets the stored weights, a per-layer hook
    (the 4-bit loader) sees each layer with its stored weights before it packs them, and shards with an index file
    work the same."""
    import json
    import os

    import torch
    from safetensors.torch import save_file

    import fms_acceleration_b200.plugins  # noqa: F401
    from fms_acceleration_b200.models.builder import build_model
    from fms_acceleration_b200.nn import Linear4bit
    from fms_acceleration_b200.plugins.peft.framework_plugin_bnb import BNBAccelerationPlugin
    from fms_acceleration_b200.plugins.peft.gptqmodel.utils.model import shard_checkpoint

    src = build_model("tiny-llama", seed=3)
    state = {k: v.contiguous() for k, v in src.state_dict().items()}
    config = {**src.config.to_dict(), "name_or_path": ""}
    one, many = tmp_path / "one", tmp_path / "many"
    os.makedirs(one)
    os.makedirs(many)
    save_file(state, str(one / "model.safetensors"), metadata={"format": "pt"})
    shards, index = shard_checkpoint(state, 200_000)
    assert len(shards) > 1
    for name, part in shards.items():
        save_file(part, str(many / name), metadata={"format": "pt"})
    json.dump(index, open(many / "model.safetensors.index.json", "w"))
    for d in (one, many):
        json.dump(config, open(d / "config.json", "w"))
        loaded = build_model(str(d))
        assert all(torch.equal(a, b) for a, b in zip(loaded.state_dict().values(), src.state_dict().values()))

    plugin = BNBAccelerationPlugin({"peft": {"quantization": {"bitsandbytes": {"quant_type": "nf4", "no_peft_model": False}}}})
    packed = plugin.model_loader(str(many), torch_dtype=torch.float32, device="cpu")
    got = packed.model.layers[1].mlp.down_proj.dequantize(dtype=torch.float32)
    want = Linear4bit.from_linear(src.model.layers[1].mlp.down_proj, "nf4", 64, torch.float32).dequantize(dtype=torch.float32)
    assert torch.equal(got, want)
    assert torch.equal(packed.model.embed_tokens.weight, src.model.embed_tokens.weight)
    assert torch.equal(packed.model.norm.weight, src.model.norm.weight)
