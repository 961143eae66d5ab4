"""ScatterMoE on CPU: checkpoint key mapping with fake weight maps, module swap parity, checkpoint round trip."""
import json

import pytest
import torch

from fms_acceleration_b200.models.builder import build_model
from fms_acceleration_b200.plugins.moe.utils import prepare_scattermoe
from fms_acceleration_b200.plugins.moe.utils import checkpoint_utils as CU
from fms_acceleration_b200.plugins.moe.utils.scattermoe_constants import (PARAM_NAME_ROUTER_SCATTERMOE,
                                                                          PARAM_NAME_WEIGHT_SCATTERMOE)
from fms_acceleration_b200.plugins.moe.utils.scattermoe_state_dict import get_checkpoint_meta_from_sharded_safetensor

F = "model-00001-of-00001.safetensors"


def _sharded_map(prefix, module, router, expert, layers, experts, keys):
    m = {}
    for i in range(layers):
        m[f"{prefix}.{i}.{module}.{router}.weight"] = F
        for j in range(experts):
            for k in keys:
                m[f"{prefix}.{i}.{module}.{expert}.{j}.{k}.weight"] = F
    return m


def _fused_map(prefix, module, router, layers, keys):
    m = {}
    for i in range(layers):
        m[f"{prefix}.{i}.{module}.{router}.weight"] = F
        for k in keys:
            m[f"{prefix}.{i}.{module}.{k}.weight"] = F
    return m


@pytest.mark.parametrize("sharded", [True, False])
def test_checkpoint_metadata_mapping(sharded):
    if sharded:
        wm = _sharded_map("model.layers", "block_sparse_moe", "gate", "experts", 2, 8, ["w1", "w2", "w3"])
        meta = get_checkpoint_meta_from_sharded_safetensor(wm, "model.layers.0", "block_sparse_moe", "gate", "experts")
    else:
        wm = _fused_map("model.layers", "block_sparse_moe", "gate", 2, ["input_linear", "output_linear"])
        meta = get_checkpoint_meta_from_sharded_safetensor(wm, "model.layers.0", "block_sparse_moe", "gate",
                                                           "input_linear|output_linear|input_linear")
    assert len(meta[f"{PARAM_NAME_ROUTER_SCATTERMOE}.weight"]) == 1
    for w in PARAM_NAME_WEIGHT_SCATTERMOE:
        assert len(meta[f"{w}.weight"]) == (8 if sharded else 1)
    if not sharded:
        assert meta["w1.weight"][0][0].endswith("input_linear.weight") and meta["w3.weight"][0][0].endswith("input_linear.weight")
        assert meta["w2.weight"][0][0].endswith("output_linear.weight")


def test_checkpoint_metadata_errors():
    wrong = {"prefix.moe_name.expert.weight": F}
    with pytest.raises(ValueError, match="Could not get safetensor map for"):
        get_checkpoint_meta_from_sharded_safetensor(wrong, "wrong_prefix", "moe_name", None, "expert_name")
    with pytest.raises(AssertionError, match="If expert_name has |, expect between 2 and"):
        get_checkpoint_meta_from_sharded_safetensor(wrong, "prefix", "moe_name", None, "exp1|exp2|exp3|exp4")
    with pytest.raises(ValueError, match="Unable to handle key 'prefix.moe_name.expert.weight'"):
        get_checkpoint_meta_from_sharded_safetensor(wrong, "prefix", "moe_name", None, "wrong_expert_name")


def test_swap_is_exact_and_converts_back(tmp_path):
    torch.manual_seed(0)
    model = build_model("tiny-granitemoe", seed=0)
    original = {k: v.clone() for k, v in model.state_dict().items()}
    ids = torch.randint(0, 1024, (2, 48))
    ref = model(ids, labels=ids).loss
    swapped = prepare_scattermoe(model, None, 0, 1, 1)
    assert len(swapped) == 2
    assert abs(model(ids, labels=ids).loss.item() - ref.item()) < 1e-5
    # ScatterMoE state -> original Hugging Face layout
    wm = {k: "model.safetensors" for k in original}
    sd = CU.recover_original_state_dict_from_checkpoint(dict(model.state_dict()), weight_map=wm,
                                                        architectures=["GraniteMoeForCausalLM"])
    assert set(sd) == set(original)
    for k in original:
        assert torch.equal(sd[k], original[k]), k


def test_dcp_save_and_recover_safetensors(tmp_path):
    from safetensors.torch import load_file, save_file

    torch.manual_seed(0)
    model = build_model("tiny-granitemoe", seed=0)
    pretrained = tmp_path / "pretrained"
    pretrained.mkdir()
    original = {k: v.clone().contiguous() for k, v in model.state_dict().items() if k != "lm_head.weight"}
    save_file(original, str(pretrained / "model.safetensors"), metadata={"format": "pt"})
    (pretrained / "config.json").write_text(json.dumps({"architectures": ["GraniteMoeForCausalLM"]}))
    prepare_scattermoe(model, None, 0, 1, 1)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-3)
    ids = torch.randint(0, 1024, (1, 32))
    model(ids, labels=ids).loss.backward()
    opt.step()
    ckpt = tmp_path / "checkpoint-1"
    ckpt.mkdir()
    CU.save_fsdp_model(None, None, model, str(ckpt), 0)
    CU.save_fsdp_optimizer(None, None, opt, model, str(ckpt), 0)
    assert (ckpt / "pytorch_model_fsdp_0").is_dir() and (ckpt / "optimizer_0").is_dir()
    out = tmp_path / "hf"
    assert CU.main([str(ckpt), str(out), str(pretrained)]) == 0
    rec = load_file(str(out / "model.safetensors"))
    trained = CU.recover_original_state_dict_from_checkpoint(
        {k: v for k, v in model.state_dict().items()}, weight_map={k: "x" for k in original},
        architectures=["GraniteMoeForCausalLM"])
    for k in original:
        assert k in rec and torch.equal(rec[k], trained[k]), k
    # resume into a fresh swapped model
    fresh = build_model("tiny-granitemoe", seed=1)
    prepare_scattermoe(fresh, None, 0, 1, 1)
    opt2 = torch.optim.AdamW(fresh.parameters(), lr=1e-3)
    fresh(ids, labels=ids).loss.backward()
    opt2.step()
    CU.load_fsdp_model(None, None, fresh, str(ckpt), 0)
    CU.load_fsdp_optimizer(None, None, opt2, fresh, str(ckpt), 0)
    for (k, a), (_, b) in zip(model.state_dict().items(), fresh.state_dict().items()):
        assert torch.equal(a, b), k


@pytest.mark.parametrize("name,arch", [("tiny-mixtral", "MixtralForCausalLM"),
                                       ("tiny-granitemoeshared", "GraniteMoeSharedForCausalLM"),
                                       ("tiny-granitemoehybrid", "GraniteMoeHybridForCausalLM")])
def test_swap_other_families(name, arch):
    """Per-expert (Mixtral) and fused (GraniteMoeShared / Hybrid) layouts convert exactly and back."""
    torch.manual_seed(0)
    model = build_model(name, seed=0)
    original = {k: v.clone() for k, v in model.state_dict().items()}
    V = model.config.vocab_size
    ids = torch.randint(0, V, (1, 40))
    cu = torch.tensor([0, 16, 40], dtype=torch.int32)
    ref = model(ids, labels=ids, cu_seqlens=cu).loss
    swapped = prepare_scattermoe(model, None, 0, 1, 1)
    assert len(swapped) == model.config.num_hidden_layers
    assert abs(model(ids, labels=ids, cu_seqlens=cu).loss.item() - ref.item()) < 1e-5
    sd = CU.recover_original_state_dict_from_checkpoint(dict(model.state_dict()),
                                                        weight_map={k: "model.safetensors" for k in original},
                                                        architectures=[arch])
    assert set(sd) == set(original)
    for k in original:
        assert torch.equal(sd[k], original[k]), k


def test_expert_lora_starts_at_the_base_and_trains_only_the_adapters():
    """Per-expert LoRA (lora_A [E, in, r] zeros, lora_B [E, r, out] normal, scale 1 as in the reference's kernels):
    the output equals the base model's at initialisation, the base expert weights are frozen, both adapter
    matrices and the router receive gradients."""
    from types import SimpleNamespace

    from fms_acceleration_b200.plugins.moe.utils.scattermoe import ScatterMoE

    torch.manual_seed(0)
    kw = dict(hidden_size=16, hidden_act="silu", intermediate_size=24, num_experts=4, top_k=2, dtype=torch.float32)
    base = ScatterMoE(**kw)
    for m in (base.w1, base.w2, base.w3):
        torch.nn.init.normal_(m.weight, std=0.2)
    torch.nn.init.normal_(base.router.weight, std=0.5)
    lora = ScatterMoE(**kw, lora_config=SimpleNamespace(r=4, lora_alpha=8))
    lora.load_state_dict(base.state_dict(), strict=False)
    x = torch.randn(10, 16)
    y0, _ = base(x)
    y1, _ = lora(x)
    assert torch.allclose(y0, y1, atol=1e-6)
    assert lora.w1.lora_A.shape == (4, 16, 4) and lora.w1.lora_B.shape == (4, 4, 24)
    assert not lora.w1.weight.requires_grad and lora.w1.lora_A.requires_grad
    with torch.no_grad():
        lora.w2.lora_A.normal_(std=0.1)          # move one adapter off zero so that lora_B sees a gradient too
    y2, _ = lora(x)
    y2.square().sum().backward()
    assert lora.w2.lora_A.grad is not None and lora.w2.lora_B.grad.abs().sum() > 0
    assert lora.w1.lora_A.grad.abs().sum() > 0 and lora.w1.weight.grad is None
    assert lora.router.weight.grad is not None
