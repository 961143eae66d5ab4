"""Hugging Face model classes through the framework on the CPU: the fused-ops plugin patches RMSNorm, rotary
embedding and the loss of a real ``transformers`` Llama, and the patched model computes what the original computes
(on the CPU every op takes its PyTorch oracle path, so this checks the plumbing: rules, triggers, replacements)."""
import copy

import pytest
import torch

transformers = pytest.importorskip("transformers")

import fms_acceleration_b200.plugins  # noqa: F401,E402  (registers the plugins)
from fms_acceleration_b200.framework.model_patcher import ModelPatcher  # noqa: E402
from fms_acceleration_b200.framework.utils.test_utils import instantiate_framework  # noqa: E402
from fms_acceleration_b200.trainer import TrainArgs  # noqa: E402


def _tiny_llama():
    # the class of the module as it is NOW: the clean-up of this test reloads the modelling module, and the
    # top-level ``transformers.LlamaForCausalLM`` may still be the class of the module before the reload
    from transformers import LlamaConfig
    from transformers.models.llama.modeling_llama import LlamaForCausalLM

    cfg = LlamaConfig(vocab_size=512, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, max_position_embeddings=128, rms_norm_eps=1e-6, tie_word_embeddings=False,
                      architectures=["LlamaForCausalLM"])
    torch.manual_seed(0)
    return LlamaForCausalLM(cfg)


@pytest.mark.parametrize("fast_loss", [True, "fused_ce_liger"])
def test_foak_patches_hf_llama_and_keeps_the_numbers(fast_loss):
    model = _tiny_llama()
    ref = copy.deepcopy(model)
    ids = torch.randint(0, 512, (2, 24))
    cfg = {"training": {"fused_ops_and_kernels": {"fused_lora": False, "fast_loss": fast_loss, "fast_rms_layernorm": True,
                                                 "fast_rope_embeddings": True}}}
    saved_rules, saved_hist = dict(ModelPatcher.rules), list(ModelPatcher.history)
    try:
        with instantiate_framework(cfg, require_packages_check=False) as fw:
            model, _ = fw.augmentation(model, TrainArgs(bf16=False), modifiable_args=(None,))
            fw.get_callbacks_and_ready_for_train(model, None)
            ModelPatcher.patch(model)
            applied = {h.rule_id for h in ModelPatcher.history}
            assert "llama-rms" in applied, applied
            assert any(r.startswith("llama-") and ("loss" in r or "lce" in r) for r in applied), applied
            model.train()
            ref.train()
            out = model(input_ids=ids, labels=ids)
            want = ref(input_ids=ids, labels=ids)
            assert torch.allclose(out.loss, want.loss, atol=1e-4, rtol=1e-4)
            out.loss.backward()
            want.loss.backward()
            g1 = model.model.layers[0].self_attn.q_proj.weight.grad
            g2 = ref.model.layers[0].self_attn.q_proj.weight.grad
            assert torch.allclose(g1, g2, atol=1e-5, rtol=1e-3)
            if fast_loss == "fused_ce_liger":
                assert out.logits is None  # the training branch never materialises the logits
    finally:
        ModelPatcher.rules.clear()
        ModelPatcher.rules.update(saved_rules)
        ModelPatcher.history[:] = saved_hist
        import importlib

        import transformers.models.llama.modeling_llama as ml

        importlib.reload(ml)


def _tiny_hf(family):
    """A two-layer model of ``family``, its class taken from the modelling module as it is now."""
    common = dict(vocab_size=512, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2)
    if family == "mistral":
        from transformers import MistralConfig as C
        from transformers.models.mistral.modeling_mistral import MistralForCausalLM as M

        cfg = C(intermediate_size=128, architectures=["MistralForCausalLM"], **common)
    elif family == "granite":
        from transformers import GraniteConfig as C
        from transformers.models.granite.modeling_granite import GraniteForCausalLM as M

        cfg = C(intermediate_size=128, architectures=["GraniteForCausalLM"], logits_scaling=4.0, embedding_multiplier=3.0,
                residual_multiplier=0.5, attention_multiplier=0.1, **common)
    elif family == "mixtral":
        from transformers import MixtralConfig as C
        from transformers.models.mixtral.modeling_mixtral import MixtralForCausalLM as M

        cfg = C(intermediate_size=96, num_local_experts=4, num_experts_per_tok=2, architectures=["MixtralForCausalLM"],
                **common)
    elif family == "granitemoeshared":
        from transformers import GraniteMoeSharedConfig as C
        from transformers.models.granitemoeshared.modeling_granitemoeshared import GraniteMoeSharedForCausalLM as M

        cfg = C(intermediate_size=96, num_local_experts=4, num_experts_per_tok=2, shared_intermediate_size=64,
                architectures=["GraniteMoeSharedForCausalLM"], **common)
    elif family == "granitemoehybrid":
        from transformers import GraniteMoeHybridConfig as C
        from transformers.models.granitemoehybrid.modeling_granitemoehybrid import GraniteMoeHybridForCausalLM as M

        cfg = C(intermediate_size=96, num_local_experts=4, num_experts_per_tok=2, shared_intermediate_size=64,
                layer_types=["mamba", "attention"], mamba_n_heads=4, mamba_d_head=32, mamba_expand=2, mamba_d_state=16,
                mamba_chunk_size=8, architectures=["GraniteMoeHybridForCausalLM"], **common)
    else:
        from transformers import GraniteMoeConfig as C
        from transformers.models.granitemoe.modeling_granitemoe import GraniteMoeForCausalLM as M

        cfg = C(intermediate_size=96, num_local_experts=4, num_experts_per_tok=2, architectures=["GraniteMoeForCausalLM"],
                **common)
    torch.manual_seed(0)
    return M(cfg)


@pytest.mark.parametrize("family", ["mistral", "granite", "mixtral", "granitemoe", "granitemoeshared", "granitemoehybrid"])
@pytest.mark.parametrize("fast_loss", [True, "fused_ce_liger"])
def test_foak_rules_of_the_other_families_keep_the_numbers(family, fast_loss):
    """RMSNorm, rotary embedding and loss rules on the Hugging Face classes of every family that has them: the
    rules apply, and loss and gradients equal the unpatched model's (Granite's logit scaling included)."""
    model = _tiny_hf(family)
    ref = copy.deepcopy(model)
    ids = torch.randint(0, 512, (2, 24))
    cfg = {"training": {"fused_ops_and_kernels": {"fused_lora": False, "fast_loss": fast_loss, "fast_rms_layernorm": True,
                                                 "fast_rope_embeddings": True}}}
    saved_rules, saved_hist = dict(ModelPatcher.rules), list(ModelPatcher.history)
    try:
        with instantiate_framework(cfg, require_packages_check=False) as fw:
            model, _ = fw.augmentation(model, TrainArgs(bf16=False), modifiable_args=(None,))
            fw.get_callbacks_and_ready_for_train(model, None)
            ModelPatcher.patch(model)
            applied = {h.rule_id for h in ModelPatcher.history}
            loss_rule = f"{family}-fused-lce" if fast_loss == "fused_ce_liger" else f"{family}-custom-loss"
            assert {f"{family}-rms", f"{family}-rope", loss_rule} <= applied, applied
            model.train()
            ref.train()
            out, want = model(input_ids=ids, labels=ids), ref(input_ids=ids, labels=ids)
            assert torch.allclose(out.loss, want.loss, atol=1e-5, rtol=1e-5)
            out.loss.backward()
            want.loss.backward()
            got = {n: p.grad for n, p in model.named_parameters() if p.grad is not None}
            exp = {n: p.grad for n, p in ref.named_parameters() if p.grad is not None}
            assert set(got) == set(exp)
            for n in exp:
                assert torch.allclose(got[n], exp[n], atol=1e-5, rtol=1e-3), n
    finally:
        ModelPatcher.rules.clear()
        ModelPatcher.rules.update(saved_rules)
        ModelPatcher.history[:] = saved_hist
        import importlib

        importlib.reload(importlib.import_module(type(ref).__module__))


@pytest.mark.parametrize("family", ["granitemoe", "mixtral", "granitemoeshared", "granitemoehybrid"])
def test_scattermoe_swaps_hf_moe_blocks_exactly_and_converts_back(family):
    """The module swap works on the installed transformers' MoE classes (fused 3-D expert parameters and hidden-only
    return value in transformers >= 5; one linear per expert and a tuple before; with a shared dense branch and with
    Mamba layers beside the attention layers), and the ScatterMoE state converts back to the original parameter names
    and values."""
    from fms_acceleration_b200.plugins.moe.utils import checkpoint_utils as CU
    from fms_acceleration_b200.plugins.moe.utils import prepare_scattermoe

    model = _tiny_hf(family).eval()
    M = type(model)
    original = {k: v.clone() for k, v in model.state_dict().items()}
    ids = torch.randint(0, 512, (2, 16))
    ref = model(input_ids=ids, labels=ids).loss
    swapped = prepare_scattermoe(model, None, 0, 1, 1)
    # the attribute name of the block inside its layer depends on the transformers version
    assert len(swapped.paths) == 2 and len(swapped) == 1 and swapped <= {"block_sparse_moe", "mlp"}
    assert abs(model(input_ids=ids, labels=ids).loss.item() - ref.item()) < 1e-5
    sd = CU.recover_original_state_dict_from_checkpoint(dict(model.state_dict()),
                                                        weight_map={k: "model.safetensors" for k in original},
                                                        architectures=[M.__name__])
    assert set(sd) == set(original)
    for k in original:
        assert torch.equal(sd[k], original[k]), k


@pytest.mark.parametrize("family", ["llama", "granitemoe"])
def test_in_tree_models_load_hf_checkpoints(tmp_path, family):
    """A checkpoint written by ``save_pretrained`` (config.json + model.safetensors) loads into the in-tree model of
    the same architecture and gives the same logits."""
    from fms_acceleration_b200.models.builder import build_model

    torch.manual_seed(0)
    if family == "llama":
        hf = _tiny_llama().eval()
    else:
        from transformers import GraniteMoeConfig, GraniteMoeForCausalLM

        hf = GraniteMoeForCausalLM(GraniteMoeConfig(
            vocab_size=512, hidden_size=64, intermediate_size=32, num_hidden_layers=2, num_attention_heads=4,
            num_key_value_heads=2, num_local_experts=4, num_experts_per_tok=2, architectures=["GraniteMoeForCausalLM"],
            tie_word_embeddings=True)).eval()
    path = tmp_path / family
    hf.save_pretrained(str(path), safe_serialization=True)
    mine = build_model(str(path), dtype=torch.float32).eval()
    ids = torch.randint(0, 512, (2, 20))
    with torch.no_grad():
        want = hf(input_ids=ids).logits
        got = mine(input_ids=ids).logits
    assert torch.allclose(got, want, atol=2e-4, rtol=1e-3), (got - want).abs().max()


def test_padding_free_plugin_routes_hf_attention_to_the_in_tree_kernel():
    """With the padding-free plugin a Hugging Face Llama runs a packed row (position ids restarting per document)
    through the registered in-tree attention and gives, per document, what the unpatched model gives on that
    document alone."""
    from fms_acceleration_b200.plugins.aadp.flash_attn import HF_ATTENTION_NAME

    model = _tiny_llama().eval()
    ref = copy.deepcopy(model)
    lens = [9, 17, 6]
    docs = [torch.randint(0, 512, (1, n)) for n in lens]
    with torch.no_grad():
        ref_logits = torch.cat([ref(input_ids=d).logits[0] for d in docs], 0)
    with instantiate_framework({"training": {"attention": {"padding_free": {"method": "huggingface"}}}},
                               require_packages_check=False) as fw:
        args = TrainArgs(padding_free=False)
        model, _ = fw.augmentation(model, args, modifiable_args=(None,))
        assert args.padding_free is True
    assert model.config._attn_implementation == HF_ATTENTION_NAME
    ids = torch.cat(docs, 1)
    pos = torch.cat([torch.arange(n) for n in lens])[None]
    with torch.no_grad():
        out = model(input_ids=ids, position_ids=pos).logits[0]
    assert torch.allclose(out, ref_logits, rtol=1e-4, atol=1e-4)
    # without position ids every row of the batch is one document: plain causal attention
    with torch.no_grad():
        a = model(input_ids=docs[1]).logits
        b = ref(input_ids=docs[1]).logits
    assert torch.allclose(a, b, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("family", ["mamba2", "granitemoehybrid"])
def test_hf_mamba_layers_swap_to_the_in_tree_mixer(family):
    """What the context-parallel plugin does to a Hugging Face model before it installs the communicator: every
    Mamba2 layer becomes the in-tree mixer with the same weights, the same parameter names and the same outputs."""
    from fms_acceleration_b200.plugins.mcp.utils.utils import swap_hf_mamba_modules

    torch.manual_seed(0)
    if family == "mamba2":
        cfg = transformers.Mamba2Config(vocab_size=256, hidden_size=64, state_size=16, num_hidden_layers=2, expand=2,
                                        head_dim=16, num_heads=8, n_groups=1, conv_kernel=4, chunk_size=32,
                                        tie_word_embeddings=False)
        model, names, expect = transformers.Mamba2ForCausalLM(cfg).eval(), ("mixer",), 2
    else:
        cfg = transformers.GraniteMoeHybridConfig(
            vocab_size=256, hidden_size=64, intermediate_size=64, num_hidden_layers=3, num_attention_heads=4,
            num_key_value_heads=2, num_local_experts=4, num_experts_per_tok=2, shared_intermediate_size=64,
            layer_types=["mamba", "attention", "mamba"], mamba_n_heads=8, mamba_d_head=16, mamba_d_state=16,
            mamba_n_groups=1, mamba_d_conv=4, mamba_expand=2, mamba_chunk_size=32, mamba_conv_bias=True,
            mamba_proj_bias=False, tie_word_embeddings=False, position_embedding_type="rope")
        model, names, expect = transformers.GraniteMoeHybridForCausalLM(cfg).eval(), ("mamba",), 2
    ids = torch.randint(0, 256, (2, 48))
    with torch.no_grad():
        ref = model(input_ids=ids).logits
    before = {k: v.clone() for k, v in model.state_dict().items()}
    assert swap_hf_mamba_modules(model, names=names) == expect
    assert swap_hf_mamba_modules(model, names=names) == 0          # already in-tree: nothing left to swap
    with torch.no_grad():
        out = model(input_ids=ids).logits
    assert torch.allclose(out, ref, rtol=1e-4, atol=1e-5)
    after = model.state_dict()
    assert sorted(after) == sorted(before) and all(torch.equal(after[k], before[k]) for k in before)
    assert not model.load_state_dict(before).missing_keys


@pytest.mark.parametrize("with_bias", [False, True])
@pytest.mark.parametrize("base", ["bitsandbytes", "auto_gptq"])
def test_fused_lora_rules_on_a_quantised_hf_llama_keep_the_numbers(base, with_bias):
    """LoRA adapters over 4-bit (NF4 / GPTQ) base layers inside a Hugging Face Llama: the fused attention and MLP
    rules fire (one projection group per fused op, the first projection called computes the group and the others read
    their slice), and loss and every adapter gradient equal the unfused model's."""
    from transformers import LlamaConfig
    from transformers.models.llama.modeling_llama import LlamaForCausalLM

    from fms_acceleration_b200.models.builder import quantize_linears_
    from fms_acceleration_b200.nn import Linear4bit, LoraConfig, get_peft_model
    from fms_acceleration_b200.nn.gptq import QuantLinear

    cfg = LlamaConfig(vocab_size=512, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, architectures=["LlamaForCausalLM"], attention_bias=with_bias,
                      mlp_bias=with_bias)
    torch.manual_seed(0)
    model = LlamaForCausalLM(cfg)
    if with_bias:
        for name, p in model.named_parameters():
            if name.endswith("proj.bias"):
                torch.nn.init.normal_(p, std=0.5)  # large enough that a dropped bias cannot go unnoticed

    def four_bit(lin):
        if base == "bitsandbytes":
            return Linear4bit.from_linear(lin, "nf4", 64, torch.float32)
        q = QuantLinear.random(lin.in_features, lin.out_features, group_size=32, dtype=torch.float32)
        if lin.bias is not None:
            q.bias = lin.bias.data.clone()
        return q

    for layer in model.model.layers:
        quantize_linears_(layer, four_bit)
    model = get_peft_model(model, LoraConfig(r=4, lora_alpha=8, lora_dropout=0.0, target_modules=[
        "q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"]))
    for name, p in model.named_parameters():
        if "lora_B" in name:
            torch.nn.init.normal_(p, std=0.05)
    model.quantization_method = "bitsandbytes" if base == "bitsandbytes" else "gptq"
    ref = copy.deepcopy(model)
    ids = torch.randint(0, 512, (2, 24))
    conf = {"peft": {"quantization": {"fused_ops_and_kernels": {"base_layer": base, "fused_lora": True, "fast_loss": True,
                                                               "fast_rms_layernorm": True, "fast_rope_embeddings": True}}}}
    saved_rules, saved_hist = dict(ModelPatcher.rules), list(ModelPatcher.history)
    try:
        with instantiate_framework(conf, require_packages_check=False) as fw:
            model, _ = fw.augmentation(model, TrainArgs(bf16=True), modifiable_args=(None,))
            fw.get_callbacks_and_ready_for_train(model, None)
            ModelPatcher.patch(model)
            applied = {h.rule_id for h in ModelPatcher.history}
            assert "llama-mlp" in applied and any(r.startswith("llama-qkvo") for r in applied), applied
            model.train()
            ref.train()
            out, want = model(input_ids=ids, labels=ids), ref(input_ids=ids, labels=ids)
            assert torch.allclose(out.loss, want.loss, atol=1e-6)
            out.loss.backward()
            want.loss.backward()
            got = {n: p.grad for n, p in model.named_parameters() if p.grad is not None}
            exp = {n: p.grad for n, p in ref.named_parameters() if p.grad is not None}
            assert set(got) == set(exp) and len(exp) == 28  # 7 projections x 2 layers x (A, B)
            for n in exp:
                assert torch.allclose(got[n], exp[n], atol=1e-6, rtol=1e-4), n
    finally:
        ModelPatcher.rules.clear()
        ModelPatcher.rules.update(saved_rules)
        ModelPatcher.history[:] = saved_hist
        import importlib

        import transformers.models.llama.modeling_llama as ml

        importlib.reload(ml)


@pytest.mark.parametrize("kind", ["nf4", "gptq", "dense"])
def test_projection_group_with_lora_dropout_matches_the_written_out_formula(kind):
    """``y = x W^T + b + s (dropout(x) A^T) B^T`` per projection: the group's autograd function keeps the dropout mask
    of its forward for its backward, the base branch sees ``x`` and the adapter branch the dropped-out ``x``."""
    from fms_acceleration_b200.nn import Linear4bit
    from fms_acceleration_b200.nn.gptq import QuantLinear
    from fms_acceleration_b200.nn.lora import LoraLinear
    from fms_acceleration_b200.ops.proj import ProjGroup
    from fms_acceleration_b200.plugins.foak.models.utils import _run_group

    torch.manual_seed(0)
    p, layers, weights = 0.25, [], []
    for out_features in (32, 16):
        lin = torch.nn.Linear(64, out_features, bias=True)
        if kind == "nf4":
            base = Linear4bit.from_linear(lin, "nf4", 64, torch.float32)
            weights.append(base.dequantize(dtype=torch.float32))
        elif kind == "gptq":
            base = QuantLinear.random(64, out_features, group_size=32, dtype=torch.float32, scale_std=0.05)
            base.bias = lin.bias.data.clone()
            weights.append(base.dequantize(dtype=torch.float32).t())
        else:
            base = lin
            base.weight.requires_grad_(False)
            weights.append(lin.weight.data)
        lora = LoraLinear(base, r=4, lora_alpha=8, lora_dropout=p)
        torch.nn.init.normal_(lora.lora_B["default"].weight, std=0.1)
        layers.append(lora.train())
    group = ProjGroup(layers, "dropout-test")
    x = torch.randn(6, 64, requires_grad=True)

    torch.manual_seed(11)
    y = _run_group(group, x)
    torch.manual_seed(11)
    keep = (torch.rand(x.shape) >= p).float() / (1.0 - p)  # the first random draw of the forward
    x_ref = x.detach().clone().requires_grad_()
    outs = []
    for lora, W in zip(layers, weights):
        A, B = lora.lora_A["default"].weight, lora.lora_B["default"].weight
        bias = lora.base_layer.bias
        outs.append(x_ref @ W.t() + bias + lora.scaling["default"] * ((x_ref * keep) @ A.t()) @ B.t())
    want = torch.cat(outs, dim=-1)
    assert torch.allclose(y, want, atol=1e-5)

    g = torch.randn_like(y)
    params = [t for lora in layers for t in (lora.lora_A["default"].weight, lora.lora_B["default"].weight)]
    got = torch.autograd.grad(y, [x] + params, g)
    exp = torch.autograd.grad(want, [x_ref] + params, g)
    for a, b in zip(got, exp):
        assert torch.allclose(a, b, atol=1e-5, rtol=1e-4)
    # in eval mode nothing is dropped
    for lora in layers:
        lora.eval()
    plain = torch.cat([lora(x) for lora in layers], dim=-1)
    assert torch.allclose(_run_group(group, x), plain, atol=1e-5)


def test_projection_group_honours_a_user_supplied_dropout_module():
    """A dropout module that is not ``nn.Dropout`` (here: a fixed mask, as the reference's own fused-ops test installs on
    every adapter) gives the same output and gradients fused and unfused."""
    from fms_acceleration_b200.nn import Linear4bit
    from fms_acceleration_b200.nn.lora import LoraLinear
    from fms_acceleration_b200.ops.proj import ProjGroup
    from fms_acceleration_b200.plugins.foak.models.utils import _run_group

    class FixedMask(torch.nn.Module):
        mask = None

        def forward(self, x):
            return x * FixedMask.mask

    torch.manual_seed(3)
    FixedMask.mask = (torch.rand(6, 64) >= 0.3).float()
    layers = []
    for out_features in (32, 16, 16):
        base = Linear4bit.from_linear(torch.nn.Linear(64, out_features, bias=False), "nf4", 64, torch.float32)
        lora = LoraLinear(base, r=4, lora_alpha=8)
        lora.lora_dropout = torch.nn.ModuleDict({"default": FixedMask()})
        torch.nn.init.normal_(lora.lora_B["default"].weight, std=0.1)
        layers.append(lora.train())
    group = ProjGroup(layers, "fixed-mask")
    x = torch.randn(6, 64, requires_grad=True)
    x_ref = x.detach().clone().requires_grad_()
    y = _run_group(group, x)
    want = torch.cat([lora(x_ref) for lora in layers], dim=-1)
    assert torch.allclose(y, want, atol=1e-5)
    params = [t for lora in layers for t in (lora.lora_A["default"].weight, lora.lora_B["default"].weight)]
    g = torch.randn_like(y)
    got = torch.autograd.grad(y, [x] + params, g)
    exp = torch.autograd.grad(want, [x_ref] + params, g)
    for a, b in zip(got, exp):
        assert torch.allclose(a, b, atol=1e-5, rtol=1e-4)
