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
    assert len(swapped.paths) == 2 and swapped == {"block_sparse_moe"}
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
    assert len(swapped.paths) == model.config.num_hidden_layers
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


def test_packed_expert_lora_reproduces_the_three_low_rank_updates():
    """pack_expert_lora: gate and up side by side, ranks padded to the kernel's 64-element contraction block; the
    packed products equal the per-projection A B and gradients flow back to the six factors."""
    from fms_acceleration_b200.ops.moe import pack_expert_lora

    torch.manual_seed(0)
    El, H, I, r = 3, 16, 24, 5
    f = [torch.randn(*s, dtype=torch.float64, requires_grad=True) for s in
         ((El, H, r), (El, r, I), (El, H, r), (El, r, I), (El, I, r), (El, r, H))]
    A13, B13, A2, B2 = pack_expert_lora(*f)
    assert A13.shape == (El, H, 64) and B13.shape == (El, 64, 2 * I) and A2.shape == (El, I, 64) and B2.shape == (El, 64, H)
    up13 = torch.bmm(A13, B13)
    assert torch.allclose(up13[:, :, :I], torch.bmm(f[0], f[1])) and torch.allclose(up13[:, :, I:], torch.bmm(f[2], f[3]))
    assert torch.allclose(torch.bmm(A2, B2), torch.bmm(f[4], f[5]))
    (up13.sum() + torch.bmm(A2, B2).sum()).backward()
    assert all(t.grad is not None and t.grad.abs().sum() > 0 for t in f)


def _emulated_grouped_gemm(a, b, seg_off, n_groups, *, mode, b_mn=True, out=None, out_dtype=None, c=None, beta=0.0,
                           n=None, m=None, b_alt=None, a2=None, b2=None, max_ctas=0):
    """Plain-torch statement of what ``ops.moe.grouped_gemm`` asks of the kernel (fp64 accumulation)."""
    off = seg_off.tolist()
    if mode == 1:
        rows, K = a.shape
        res = torch.zeros(rows, n, dtype=torch.float64)
        for g in range(n_groups):
            r0, r1 = off[g], off[g + 1]

            def weight(t, kk, cols):
                if b_mn:
                    return t[g * kk:(g + 1) * kk, :cols].double()            # stored [K, N]
                return t[g * cols:(g + 1) * cols, :kk].double().t()          # stored [N, K]

            if b_alt is not None:
                half = b.shape[1]
                res[r0:r1, :half] = a[r0:r1].double() @ weight(b, K, half)
                res[r0:r1, half:] = a[r0:r1].double() @ weight(b_alt, K, half)
            else:
                res[r0:r1] = a[r0:r1].double() @ weight(b, K, n)
            if a2 is not None:
                res[r0:r1] += a2[r0:r1].double() @ weight(b2, a2.shape[1], n)
        if c is not None:
            res += beta * c.double()
        res = res.to(out_dtype or (out.dtype if out is not None else a.dtype))
        if out is not None:
            out.copy_(res)
            return out
        return res
    res = torch.zeros(n_groups, m, n, dtype=torch.float64)
    for g in range(n_groups):
        r0, r1 = off[g], off[g + 1]
        res[g] = a[r0:r1].double().t() @ b[r0:r1].double()
    if c is not None:
        res += beta * c.double()
    res = res.to(out_dtype or torch.float32)
    if out is not None:
        out.copy_(res)
        return out
    return res


def test_expert_lora_gradient_algebra_against_autograd(monkeypatch):
    """The chain of grouped products that carries per-expert LoRA through the expert MLP (forward and backward of
    ops.moe._experts_fwd_local / _experts_bwd_local), with the kernel calls replaced by plain torch: outputs, the
    input gradient and the gradients of the four packed factors equal autograd's on the dense W + A B formulation."""
    from types import SimpleNamespace

    from fms_acceleration_b200.ops import moe as MOE

    torch.manual_seed(0)
    El, H, I, r = 3, 16, 24, 4
    counts = [5, 0, 9]
    off = [0]
    for cnt in counts:
        off.append(off[-1] + cnt)
    rows = off[-1]
    seg_off = torch.tensor(off + [rows], dtype=torch.int32)
    dd = torch.float64

    def glu_fwd(e, g, act, rows_dev=None):
        return torch.nn.functional.silu(e) * g

    def glu_bwd(dh, e, g, act, de=None, dg=None, rows_dev=None):
        sig = torch.sigmoid(e)
        d_e = dh * g * (sig * (1 + e * (1 - sig)))
        d_g = dh * torch.nn.functional.silu(e)
        de.copy_(d_e)
        dg.copy_(d_g)

    monkeypatch.setattr(MOE, "grouped_gemm", _emulated_grouped_gemm)
    monkeypatch.setattr(MOE.ACT, "glu_fwd", glu_fwd)
    monkeypatch.setattr(MOE.ACT, "glu_bwd", glu_bwd)
    mctx = SimpleNamespace(I=I, E_local=El, H=H, gemm_ctas=0)
    w1, w3 = torch.randn(El, H, I, dtype=dd) * 0.3, torch.randn(El, H, I, dtype=dd) * 0.3
    w2 = torch.randn(El, I, H, dtype=dd) * 0.3
    fac = [(torch.randn(*s, dtype=dd) * 0.3).requires_grad_() for s in
           ((El, H, r), (El, r, I), (El, H, r), (El, r, I), (El, I, r), (El, r, H))]
    lora = MOE.pack_expert_lora(*fac)
    Xs = torch.randn(rows, H, dtype=dd)
    dYs = torch.randn(rows, H, dtype=dd)
    packed = tuple(t.detach() for t in lora)
    gu, Ys, XA = MOE._experts_fwd_local(mctx, Xs, seg_off, w1, w3, w2, "silu", lora=packed)
    acc: dict = {}
    dXs = MOE._experts_bwd_local(mctx, Xs, gu, dYs, seg_off, w1, w3, w2, "silu", acc, need_dw=False, lora=packed, XA=XA)

    xs = Xs.clone().requires_grad_()
    ref = torch.zeros(rows, H, dtype=dd)
    for g in range(El):
        r0, r1 = off[g], off[g + 1]
        d1, d3, d2 = w1[g] + fac[0][g] @ fac[1][g], w3[g] + fac[2][g] @ fac[3][g], w2[g] + fac[4][g] @ fac[5][g]
        ref[r0:r1] = (torch.nn.functional.silu(xs[r0:r1] @ d1) * (xs[r0:r1] @ d3)) @ d2
    assert torch.allclose(Ys, ref.detach(), atol=1e-9)
    ref.backward(dYs)
    assert torch.allclose(dXs, xs.grad, atol=1e-9)
    got = dict(zip(("da13", "db13", "da2", "db2"), (acc[k].double() for k in ("da13", "db13", "da2", "db2"))))
    # autograd through the packing gives the reference gradients of the packed tensors
    pk = [t.detach().clone().requires_grad_() for t in lora]
    xs2 = Xs.clone()
    ref2 = torch.zeros(rows, H, dtype=dd)
    for g in range(El):
        r0, r1 = off[g], off[g + 1]
        up = torch.cat([w1[g], w3[g]], dim=1) + pk[0][g] @ pk[1][g]
        hid = torch.nn.functional.silu(xs2[r0:r1] @ up[:, :I]) * (xs2[r0:r1] @ up[:, I:])
        ref2[r0:r1] = hid @ (w2[g] + pk[2][g] @ pk[3][g])
    ref2.backward(dYs)
    for key, t in zip(("da13", "db13", "da2", "db2"), pk):
        assert torch.allclose(got[key], t.grad, atol=1e-5), key


def test_all_linear_given_as_a_one_element_list_targets_every_linear():
    """``--target_modules all-linear`` arrives from a command line as ``["all-linear"]``."""
    import torch

    from fms_acceleration_b200.models.builder import build_model
    from fms_acceleration_b200.nn import LoraConfig, get_peft_model
    from fms_acceleration_b200.nn.lora import LoraLinear

    as_list = get_peft_model(build_model("tiny-llama", seed=0), LoraConfig(r=2, lora_alpha=4, target_modules=["all-linear"]))
    as_text = get_peft_model(build_model("tiny-llama", seed=0), LoraConfig(r=2, lora_alpha=4, target_modules="all-linear"))
    names = lambda m: sorted(n for n, mod in m.named_modules() if isinstance(mod, LoraLinear))  # noqa: E731
    assert names(as_list) == names(as_text) and len(names(as_list)) == 7 * 2  # 7 projections x 2 layers, no lm_head
    assert not any("lm_head" in n for n in names(as_list))
    ids = torch.randint(0, 100, (1, 8))
    assert torch.isfinite(as_list(ids, labels=ids).loss)


def test_cli_checkpoint_of_a_preset_run_converts_back_to_the_original_layout(tmp_path):
    """Train a ScatterMoE model that started from an architecture preset, save through the trainer CLI, convert with
    the checkpoint tool (the preset name stands in for the original checkpoint) and load the result into the plain
    model: every parameter is there under its original name."""
    import os

    import torch
    from safetensors.torch import load_file

    from fms_acceleration_b200.benchmarks import sft_trainer as T
    from fms_acceleration_b200.framework import AccelerationFramework
    from fms_acceleration_b200.framework.model_patcher import ModelPatcher
    from fms_acceleration_b200.models.builder import build_model
    from fms_acceleration_b200.plugins.moe.utils import checkpoint_utils as CU

    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = os.path.join(here, "sample-configurations", "moe-scattermoe-granite-ep1-sample-configuration.yaml")
    saved = (dict(ModelPatcher.rules), list(ModelPatcher.history))
    try:
        AccelerationFramework.reset()
        assert T.main(["--model_name_or_path", "tiny-granitemoe", "--acceleration_framework_config_file", cfg,
                       "--torch_dtype", "float32", "--bf16", "True", "--max_steps", "2", "--logging_steps", "1",
                       "--per_device_train_batch_size", "2", "--max_seq_length", "32", "--save_strategy", "epoch",
                       "--output_dir", str(tmp_path / "run")]) == 0
    finally:
        AccelerationFramework.reset()
        ModelPatcher.rules.clear()
        ModelPatcher.rules.update(saved[0])
        ModelPatcher.history[:] = saved[1]
    assert CU.main([str(tmp_path / "run" / "checkpoint-2"), str(tmp_path / "hf"), "tiny-granitemoe"]) == 0
    sd = load_file(str(tmp_path / "hf" / "model.safetensors"))
    plain = build_model("tiny-granitemoe", seed=0)
    before = {k: v.clone() for k, v in plain.state_dict().items()}
    missing, unexpected = plain.load_state_dict(sd, strict=False)
    assert not missing and not unexpected
    assert any(not torch.equal(before[k], v) for k, v in plain.state_dict().items())  # trained values, not the init
