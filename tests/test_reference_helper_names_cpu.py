"""Helper functions that code written against the reference's packages may call (CLI helpers, GPTQ utilities,
functional fused linear + cross-entropy, multipack bin packing, ScatterMoE operators, MegaBlocks-style row
permutations, Mamba-CP and data-mixing hooks): they exist under the alias packages and compute what their names say,
checked against plain PyTorch / NumPy statements on the CPU."""
import hashlib
import json
import os
import types

import numpy as np
import pytest
import torch


# ---------------------------------------------------------------------------------------------------- GPTQ utilities
def test_gptq_device_and_hash_helpers(tmp_path):
    from fms_acceleration_peft.gptqmodel.utils.model import (get_device, move_to, nested_move_to, verify_model_hash,
                                                             verify_sharded_model_hashes)

    lin = torch.nn.Linear(2, 2)
    assert get_device(lin) == torch.device("cpu") and get_device(torch.zeros(1)) == torch.device("cpu")
    assert move_to(torch.ones(2), "cpu").device.type == "cpu"
    moved = nested_move_to({"a": [torch.ones(1), (torch.zeros(1), 3)], "b": "text"}, "cpu")
    assert moved["b"] == "text" and moved["a"][1][1] == 3 and torch.equal(moved["a"][0], torch.ones(1))

    blob = tmp_path / "model-00001.safetensors"
    blob.write_bytes(b"packed weights")
    digest = hashlib.sha256(b"packed weights").hexdigest()
    assert verify_model_hash(str(blob), f"sha256:{digest}")
    assert not verify_model_hash(str(blob), "sha256:" + "0" * 64)
    index = tmp_path / "model.safetensors.index.json"
    index.write_text(json.dumps({"weight_map": {"w": blob.name}}))
    assert verify_sharded_model_hashes(str(index), [f"sha256:{digest}"])
    assert not verify_sharded_model_hashes(str(index), ["sha256:" + "1" * 64])


def test_gptq_model_type_post_init_and_configs(tmp_path):
    from fms_acceleration_peft.gptqmodel.models._const import EXPERT_INDEX_PLACEHOLDER, SUPPORTED_MODELS
    from fms_acceleration_peft.gptqmodel.models.llama import LlamaGPTQ
    from fms_acceleration_peft.gptqmodel.models.mixtral import MixtralGPTQ
    from fms_acceleration_peft.gptqmodel.quantization.config import BaseQuantizeConfig, QuantizeConfig
    from fms_acceleration_peft.gptqmodel.utils.model import (check_and_get_model_type, gptqmodel_post_init,
                                                             select_quant_linear_with_pack)
    from fms_acceleration_peft.gptqmodel.utils.peft import GPTQLoraConfig
    from fms_acceleration_b200.nn.gptq import QuantLinear

    (tmp_path / "config.json").write_text(json.dumps({"model_type": "llama"}))
    assert check_and_get_model_type(str(tmp_path)) == "llama"
    (tmp_path / "config.json").write_text(json.dumps({"model_type": "not-a-model"}))
    with pytest.raises(TypeError):
        check_and_get_model_type(str(tmp_path))
    assert "llama" in SUPPORTED_MODELS and "dbrx" not in SUPPORTED_MODELS
    assert LlamaGPTQ.layers_node == "model.layers"
    assert any(EXPERT_INDEX_PLACEHOLDER in m for group in MixtralGPTQ.layer_modules for m in group)
    assert select_quant_linear_with_pack(4, 128, False, True) is QuantLinear
    model = torch.nn.Sequential(QuantLinear.random(64, 32, group_size=32, dtype=torch.float32))
    assert gptqmodel_post_init(model) is model
    assert issubclass(BaseQuantizeConfig, QuantizeConfig)
    cfg = GPTQLoraConfig(r=4, lora_alpha=8, target_modules=["q_proj"])
    assert cfg.injected_fused_attention is False and cfg.injected_fused_mlp is False and cfg.r == 4


def test_gptq_function_forms_and_linear_view():
    from fms_acceleration_foak.fused_ops.unsloth_lora.gptq.triton.layers import GPTQuantLinear
    from fms_acceleration_peft.gptqmodel.nn_modules.triton_utils.dequant import QuantLinearFunction
    from fms_acceleration_peft.gptqmodel.nn_modules.triton_utils.kernels import (
        QuantLinearInferenceOnlyFunction, quant_matmul_248, transpose_quant_matmul_248)
    from fms_acceleration_peft.gptqmodel.nn_modules.triton_utils.mixin import TritonModuleMixin
    from fms_acceleration_b200.nn.gptq import QuantLinear

    torch.manual_seed(0)
    q = QuantLinear.random(128, 64, group_size=32, dtype=torch.float32)
    W = q.dequantize(dtype=torch.float32)
    x = torch.randn(5, 128, requires_grad=True)
    args = (q.qweight, q.scales, q.qzeros, q.g_idx, q.bits, 15)
    assert torch.allclose(quant_matmul_248(x, *args), x @ W, atol=1e-4)
    dy = torch.randn(5, 64)
    assert torch.allclose(transpose_quant_matmul_248(dy, *args), dy @ W.t(), atol=1e-4)
    y = QuantLinearFunction.apply(x, *args)
    y.backward(dy)
    assert torch.allclose(x.grad, dy @ W.t(), atol=1e-4)
    assert not QuantLinearInferenceOnlyFunction.apply(x, *args).requires_grad
    assert TritonModuleMixin.warmup(None) is None

    holder = torch.nn.Sequential(q)
    want = q(x.detach())
    assert GPTQuantLinear.inject_to_model(holder, QuantLinear) == 1
    assert isinstance(holder[0], torch.nn.Linear) and holder[0].qweight is q.qweight
    assert torch.allclose(holder(x.detach()), want, atol=1e-5)
    frozen = GPTQuantLinear(q, trainable=False)
    assert not frozen(x).requires_grad


def test_autogptq_utils_float_view_and_all_linear():
    import fms_acceleration_peft.autogptq_utils as U
    from fms_acceleration_b200.nn.gptq import QuantLinear

    cfg = types.SimpleNamespace(target_modules="all-linear")
    assert U.requires_installation_on_all_linears(cfg)
    cfg.target_modules = ["all-linear"]
    assert U.requires_installation_on_all_linears(cfg)
    cfg.target_modules = ["q_proj", "all-linear"]
    with pytest.raises(ValueError):
        U.requires_installation_on_all_linears(cfg)
    cfg.target_modules = ["q_proj"]
    assert not U.requires_installation_on_all_linears(cfg)
    cfg.target_modules = None
    assert not U.requires_installation_on_all_linears(cfg, "llama")
    with pytest.raises(ValueError):
        U.requires_installation_on_all_linears(cfg, "no-such-type")

    torch.manual_seed(1)
    q = QuantLinear.random(64, 32, group_size=32, dtype=torch.float32)
    x = torch.randn(3, 64)
    want = q(x)
    fwd = U.build_patch_to_view_tensor_to_parameter_for_fsdp_gptq(q, torch.float32)
    # what a float-only sharding wrapper sees: frozen float parameters
    params = dict(q.named_parameters())
    assert set(params) == {"qweight", "qzeros"}
    assert all(p.dtype == torch.float32 and not p.requires_grad for p in params.values())
    assert torch.equal(fwd(q, x), want)

    # placing a LoRA layer over a quantised one
    q2 = QuantLinear.random(64, 32, group_size=32, dtype=torch.float32)
    lora_cfg = types.SimpleNamespace(r=4, lora_alpha=8, lora_dropout=0.0)
    new = U.create_new_module_peft(lora_cfg, "default", q2, QuantLinear)
    assert new is not None and new.base_layer is q2
    assert U.create_new_module_peft(lora_cfg, "default", torch.nn.Linear(2, 2), QuantLinear) is None
    parent = torch.nn.Module()
    parent.proj = q2
    U.replace_module_peft(None, parent, "proj", new, q2)
    assert parent.proj is new

    meta = QuantLinear(4, 32, 64, 32, bias=True, dtype=torch.float32)
    meta._buffers["bias"] = torch.empty(32, device="meta")
    U.make_sure_no_tensor_in_meta_device(torch.nn.Sequential(meta))
    assert meta.bias.device.type == "cpu" and float(meta.bias.abs().sum()) == 0.0


# ------------------------------------------------------------------------------------------------------- fused ops
@pytest.mark.parametrize("smoothing,with_bias,reduction", [(0.0, False, "mean"), (0.1, True, "mean"), (0.0, True, "sum")])
def test_functional_fused_linear_cross_entropy(smoothing, with_bias, reduction):
    from fms_acceleration_foak.fused_ops.liger_ce.fused_linear_cross_entropy_loss import (
        fused_linear_cross_entropy_backward, fused_linear_cross_entropy_forward)

    torch.manual_seed(3)
    x = torch.randn(19, 8, requires_grad=True)
    w = torch.randn(13, 8, requires_grad=True)
    b = torch.randn(13, requires_grad=True) if with_bias else None
    t = torch.randint(0, 13, (19,))
    t[[2, 7]] = -100
    loss, gx, gw, gb = fused_linear_cross_entropy_forward(x.detach(), w.detach().requires_grad_(), t,
                                                          None if b is None else b.detach(), -100, smoothing, reduction)
    want = torch.nn.functional.cross_entropy(torch.nn.functional.linear(x, w, b), t, ignore_index=-100,
                                             label_smoothing=smoothing, reduction=reduction)
    grads = torch.autograd.grad(want, [x, w] + ([b] if with_bias else []))
    assert torch.allclose(loss, want, atol=1e-5)
    assert torch.allclose(gx, grads[0], atol=1e-5) and torch.allclose(gw, grads[1], atol=1e-5)
    if with_bias:
        assert torch.allclose(gb, grads[2], atol=1e-5)
    sx, sw, sb = fused_linear_cross_entropy_backward(torch.tensor(2.0), gx.clone(), gw.clone(), None if gb is None else gb.clone())
    assert torch.allclose(sx, 2 * grads[0], atol=1e-5) and torch.allclose(sw, 2 * grads[1], atol=1e-5)


def test_canonicalized_lora_matmul_and_activation_key():
    from fms_acceleration_foak.fused_ops.unsloth_lora.gptq.fast_lora import matmul_lora_canonicalized
    from fms_acceleration_foak.models.utils import get_hidden_activation_fn_key, get_transformers_version

    torch.manual_seed(0)
    X, W = torch.randn(2, 5, 8), torch.randn(8, 6)  # W already [in, out]
    A, B = torch.randn(3, 8), torch.randn(6, 3)
    y = matmul_lora_canonicalized(X, W, A, B, 0.5)
    assert torch.allclose(y, X @ W + 0.5 * (X @ A.t()) @ B.t(), atol=1e-5)
    assert get_hidden_activation_fn_key(types.SimpleNamespace(hidden_act="silu")) == "silu"
    assert get_hidden_activation_fn_key(types.SimpleNamespace(activation_function="gelu")) == "gelu"
    with pytest.raises(ValueError):
        get_hidden_activation_fn_key(types.SimpleNamespace(architectures=["X"]))
    assert get_transformers_version() is not None


# ------------------------------------------------------------------------------------------------------- multipack
def test_first_fit_decreasing_helpers():
    from fms_acceleration_aadp.multipack_sampler import (ffd_check, ffd_check_padding, ffd_with_result,
                                                         ffd_with_result_padding, find_padding_max_batch_len_addition,
                                                         guess_starting_avg_padding, simulate_buckets)

    a = np.array([7, 5, 4, 3, 1])
    assert ffd_check(a, 10, 2) and not ffd_check(a, 10, 1) and not ffd_check(a, 6, 10)  # 7 fits nowhere at capacity 6
    bins = ffd_with_result(a, 10, start_index=100)
    assert sorted(i for b in bins for i in b) == [100, 101, 102, 103, 104]
    assert all(sum(int(a[i - 100]) for i in b) <= 10 for b in bins) and len(bins) == 2
    # padded cost of a bin = its longest sample times its size
    padded = ffd_with_result_padding(a, 10, start_index=0)
    assert sorted(i for b in padded for i in b) == [0, 1, 2, 3, 4]
    assert all(max(int(a[i]) for i in b) * len(b) <= 10 for b in padded)
    assert ffd_check_padding(a, 10, len(padded)) and not ffd_check_padding(a, 10, 1)

    rng = np.random.default_rng(0)
    lengths = rng.integers(20, 200, size=400)
    base_avg = float(lengths.mean())
    start = guess_starting_avg_padding(base_avg, 64, 2, 1, sorted(lengths.tolist(), reverse=True))
    assert start >= 0
    few = simulate_buckets(base_avg, 64, 2, 1, 0, 10 ** 9, lengths, 0, None, 0)
    many = simulate_buckets(base_avg, 64, 2, 1, 0, 10 ** 9, lengths, 0, None, start)
    assert many >= few > 0
    dataset = [{"input_ids": [0] * int(n)} for n in lengths]
    add = find_padding_max_batch_len_addition(base_avg, 64, dataset, 2, 1, 0, 10 ** 9, 0)
    # the search stops once the simulated samples per step are within max(10, 2 %) of the goal
    reached = simulate_buckets(base_avg, 64, 2, 1, 0, 10 ** 9, lengths, 0, None, add)
    assert add > 0 and abs(reached - 64) <= 10 and reached > few


# ---------------------------------------------------------------------------------------------- ScatterMoE operators
def _routing(T, E, k, seed=0):
    torch.manual_seed(seed)
    gates, idx = torch.topk(torch.softmax(torch.randn(T, E, dtype=torch.float64), -1), k)
    sorted_experts, order = torch.sort(idx.flatten())
    return gates, idx, sorted_experts, order


def test_padded_block_indices_and_bins():
    from fms_acceleration_moe.utils.scattermoe_utils.expert_parallel import no_indices_just_bins
    from fms_acceleration_moe.utils.scattermoe_utils.khd.kernels.ops import padded_block_indices

    _, idx, se, _ = _routing(37, 5, 2)
    starts, ends = padded_block_indices(se, 5, N_BLOCK_SIZE=4)
    counts = se.bincount(minlength=5)
    want, first = [], 0
    for c in counts.tolist():
        want += [first + 4 * b for b in range((c + 3) // 4)]
        first += c
    assert starts.tolist() == want and ends.tolist() == counts.cumsum(0).tolist()
    bins, per_expert = no_indices_just_bins(idx, 5)
    assert per_expert.tolist() == counts.tolist() and bins.tolist() == ends.tolist()
    # an expert without rows contributes no tile
    starts, ends = padded_block_indices(torch.tensor([0, 0, 3]), 4, N_BLOCK_SIZE=128)
    assert starts.tolist() == [0, 2] and ends.tolist() == [2, 2, 2, 3]


def test_scattered_experts_operator_matches_a_per_token_loop():
    from fms_acceleration_moe.utils.scattermoe_utils.khd.kernels.ops import padded_block_indices, scattered_experts

    T, H, I, E, k, r = 23, 12, 20, 5, 2, 4
    gates, idx, se, ss = _routing(T, E, k, seed=1)
    gates = gates.detach().requires_grad_()
    x = torch.randn(T, H, dtype=torch.float64, requires_grad=True)
    W1 = (torch.randn(E, H, I, dtype=torch.float64) * 0.3).requires_grad_()
    W2 = torch.randn(E, I, H, dtype=torch.float64) * 0.3
    A = torch.randn(E, I, r, dtype=torch.float64, requires_grad=True)
    B = torch.randn(E, r, H, dtype=torch.float64, requires_grad=True)
    pb, eo = padded_block_indices(se, E)
    h = scattered_experts(x, W1, k, se, ss, pb, eo, grouped_out=True)
    y = scattered_experts(torch.tanh(h), W2, 1, se, ss, pb, eo, gates=gates, grouped_in=True, expert_lora_A=A,
                          expert_lora_B=B, lora_alp=2.0 * r)
    want = torch.zeros(T, H, dtype=torch.float64)
    rows = []
    for t in range(T):
        acc = 0
        for j in range(k):
            e = int(idx[t, j])
            acc = acc + gates[t, j] * (torch.tanh(x[t] @ W1[e]) @ (W2[e] + 2.0 * A[e] @ B[e]))
        rows.append(acc)
    want = torch.stack(rows)
    assert torch.allclose(y, want, atol=1e-10)
    g = torch.randn_like(y)
    got = torch.autograd.grad(y, [x, W1, gates, A, B], g, retain_graph=True)
    ref = torch.autograd.grad(want, [x, W1, gates, A, B], g)
    for a, b in zip(got, ref):
        assert torch.allclose(a, b, atol=1e-9)
    # rows scattered back into (token, choice) order without gates
    flat = scattered_experts(x, W1, k, se, ss, pb, eo)
    assert torch.allclose(flat.view(T, k, I)[3, 1], x[3] @ W1[int(idx[3, 1])], atol=1e-10)


def test_scattered_experts_module_forward_composes_like_the_reference():
    from fms_acceleration_moe.utils.scattermoe import ScatterMoE
    from fms_acceleration_moe.utils.scattermoe_utils.khd.kernels.ops import padded_block_indices

    torch.manual_seed(2)
    moe = ScatterMoE(16, "silu", 24, 4, top_k=2, dtype=torch.float32)
    for p in moe.parameters():
        torch.nn.init.normal_(p, std=0.2)
    x = torch.randn(9, 16)
    want = moe(x)
    want = want[0] if isinstance(want, tuple) else want
    _, w, idx = moe._compute_routing_weights(x)
    se, ss = torch.sort(idx.flatten().long())
    pb, eo = padded_block_indices(se, 4)
    h = torch.nn.functional.silu(moe.w1(x, se, ss, pb, eo)) * moe.w3(x, se, ss, pb, eo)
    y = moe.w2(h, se, ss, pb, eo, gates=w.to(h.dtype))
    assert torch.allclose(y, want.reshape(9, 16), atol=1e-4)


def test_building_block_ops_write_into_their_out_argument():
    from fms_acceleration_moe.utils.scattermoe_utils.khd.custom_op import torch_custom_op
    from fms_acceleration_moe.utils.scattermoe_utils.khd.kernels.ops.compileable_ops import (compileable_bincount, group,
                                                                                                  group_bwd_W)

    _, idx, se, ss = _routing(11, 3, 2, seed=4)
    A = torch.randn(11, 6, dtype=torch.float64)
    coeff = torch.rand(22, dtype=torch.float64)
    out = torch.empty(22, 6, dtype=torch.float64)
    group(A, ss, out, coeff=coeff, fan_out=2)
    assert torch.allclose(out[5], A[int(ss[5]) // 2] * coeff[int(ss[5])])
    dy = torch.randn(22, 4, dtype=torch.float64)
    ends = se.bincount(minlength=3).cumsum(0)
    dW = torch.full((3, 6, 4), 7.0, dtype=torch.float64)
    group_bwd_W(dy, out, ends, dW, 3)
    s, e = int(ends[0]), int(ends[1])
    assert torch.allclose(dW[1], out[s:e].t() @ dy[s:e])
    assert compileable_bincount(se, 3).tolist() == se.bincount(minlength=3).tolist()

    @torch_custom_op("fmsb_test::twice", mutates_args={"out"})
    def twice(x: torch.Tensor, out: torch.Tensor) -> None:
        out.copy_(2 * x)

    buf = torch.empty(3)
    twice(torch.ones(3), buf)
    assert buf.tolist() == [2.0, 2.0, 2.0]


# ------------------------------------------------------------------------------------- MegaBlocks-style permutations
def test_gather_scatter_rows_and_their_gradients():
    from fms_acceleration_moe.utils.scattermoe_utils.megablocks import autograd as MB
    from fms_acceleration_moe.utils.scattermoe_utils.megablocks.kernels import gather_scatter as K

    T, H, E, k = 7, 5, 3, 2
    gates, idx, bin_ids, indices = _routing(T, E, k, seed=5)
    bins = bin_ids.bincount(minlength=E).cumsum(0)
    x = torch.randn(T, H, dtype=torch.float64, requires_grad=True)
    w = gates.detach().flatten().requires_grad_()

    rows = K.gather(x, indices, bin_ids, None, bins, k)
    assert torch.equal(rows, x[indices // k])
    # padded layout: every bin starts at a multiple of 4 rows; padding rows are zero
    padded_bins = ((bin_ids.bincount(minlength=E) + 3) // 4 * 4).cumsum(0)
    prow = K.padded_gather(x, indices, bin_ids, None, bins, padded_bins, k)
    assert prow.shape[0] == int(padded_bins[-1])
    first_of_bin1 = int(padded_bins[0])
    assert torch.equal(prow[first_of_bin1], rows[int(bins[0])])
    back = K.padded_scatter(prow, indices, bin_ids, w, bins, padded_bins, k)
    want = (x[:, None, :] * w.view(T, k, 1)).sum(1)
    assert torch.allclose(back, want)

    # differentiable forms against index arithmetic written with autograd-aware tensor ops
    y = MB.scatter(MB.gather(x, indices, bin_ids, bins, k) * 3.0, indices, bin_ids, w, bins, k)
    ref = (3.0 * x[:, None, :] * w.view(T, k, 1)).sum(1)
    assert torch.allclose(y, ref)
    g = torch.randn_like(y)
    got = torch.autograd.grad(y, [x, w], g)
    exp = torch.autograd.grad(ref, [x, w], g)
    assert torch.allclose(got[0], exp[0]) and torch.allclose(got[1], exp[1])
    wg = K.scatter_wgrad(rows.detach(), g, indices, bin_ids, bins, k)
    assert torch.allclose(wg, (x.detach()[:, None, :] * g[:, None, :]).sum(-1).expand(T, k).flatten())
    with pytest.raises(ValueError):
        K.gather(x, indices[:-1], bin_ids, None, bins, k)


# ------------------------------------------------------------------------------------------- MoE loading / optimizer
def test_expert_loading_and_full_state_dict_helpers():
    from fms_acceleration_moe.utils import patch_torch_optim_foreach_to_not_apply_to_dtensors
    from fms_acceleration_moe.utils.checkpoint_utils import fsdp2_load_full_state_dict, fsdp2_prepare_model
    from fms_acceleration_moe.utils.scattermoe import ScatterMoE
    from fms_acceleration_moe.utils.scattermoe_prepare import load_experts_onto_device
    from torch.optim import optimizer as opt_mod

    patch_torch_optim_foreach_to_not_apply_to_dtensors()
    assert all(t.__name__ != "DTensor" for t in getattr(opt_mod, "_foreach_supported_types", []))
    assert patch_torch_optim_foreach_to_not_apply_to_dtensors() == 0

    moe = ScatterMoE(8, "silu", 4, 4, top_k=2, dtype=torch.float32)
    sd = {"router.weight": torch.full((4, 8), 0.5), "w1.weight": torch.full((4, 8, 4), 2.0),
          "w2.weight": torch.full((4, 4, 8), 3.0)}
    assert load_experts_onto_device(moe, sd) is moe
    assert float(moe.router.weight.detach().mean()) == 0.5 and float(moe.w1.weight.detach().mean()) == 2.0
    assert float(moe.w2.weight.detach().mean()) == 3.0
    # a checkpoint that holds more experts than this module owns: the module keeps its slice (rank 0 without a group)
    big = {"w1.weight": torch.arange(8.0).view(8, 1, 1).expand(8, 8, 4).contiguous()}
    load_experts_onto_device(moe, big, None, num_experts_per_device=4)
    assert moe.w1.weight[:, 0, 0].tolist() == [0.0, 1.0, 2.0, 3.0]

    lin = torch.nn.Linear(3, 2)
    fsdp2_load_full_state_dict(None, lin, {"weight": torch.zeros(2, 3), "bias": torch.ones(2)})
    assert float(lin.weight.detach().abs().sum()) == 0.0 and float(lin.bias.detach().sum()) == 2.0
    assert fsdp2_prepare_model(None, lin) is lin


# ------------------------------------------------------------------------------------------- Mamba-CP and ODM hooks
def test_mamba_cp_and_data_mixing_hook_names():
    import fms_acceleration_mcp.utils.utils as MU
    from fms_acceleration_odm import patch as OP
    from fms_acceleration_b200.models.mamba2 import Mamba2Mixer

    cfg = types.SimpleNamespace(hidden_size=64, mamba_n_groups=1, mamba_chunk_size=64, mamba_conv_bias=True, mamba_d_conv=4)
    ssm = MU.get_ssmconfig_from_hfconfig(cfg)
    assert ssm["d_model"] == 64 and ssm["d_state"] == 128 and ssm["rmsnorm"] is True and ssm["d_conv"] == 4
    assert issubclass(MU.Mamba2CPHF, Mamba2Mixer)
    with pytest.raises(AttributeError):
        MU.no_such_name  # noqa: B018

    loader = object()
    assert OP.skip_first_batches(loader, 5) is loader


def test_train_dataloader_hook_restores_the_saved_state(tmp_path):
    from fms_acceleration_odm import patch as OP
    from fms_acceleration_odm.callback import STATE_FILE

    class Loader:
        def __init__(self):
            self.state = None

        def load_state_dict(self, sd):
            self.state = sd

    class FakeTrainer:
        train_dataset = [1, 2, 3]
        _train_batch_size = 1
        _get_train_sampler = None

        def __init__(self, resume):
            self.model = types.SimpleNamespace(resume_from_checkpoint=resume)
            self.args = types.SimpleNamespace(output_dir=str(tmp_path))

        def _get_dataloader(self, **kwargs):
            assert kwargs["description"] == "Training" and kwargs["is_training"]
            return Loader()

    assert OP.get_train_dataloader(FakeTrainer(None)).state is None
    ckpt = tmp_path / "checkpoint-5"
    os.makedirs(ckpt)
    torch.save({"position": 17}, ckpt / STATE_FILE)
    assert OP.get_train_dataloader(FakeTrainer(str(ckpt))).state == {"position": 17}
    # True = the last checkpoint under the output directory
    tr = FakeTrainer(True)
    assert OP.get_train_dataloader(tr).state == {"position": 17} and tr.model.resume_from_checkpoint == str(ckpt)
    empty = FakeTrainer(True)
    empty.args.output_dir = str(tmp_path / "nothing-here")
    os.makedirs(empty.args.output_dir)
    with pytest.raises(ValueError):
        OP.get_train_dataloader(empty)
    bare = FakeTrainer(None)
    bare.train_dataset = None
    with pytest.raises(ValueError):
        OP.get_train_dataloader(bare)


# ------------------------------------------------------------------------------------------------------------ CLI
def test_cli_helper_names(tmp_path):
    from fms_acceleration.cli import get_benchmark_artifacts, install_plugin

    # the plugins ship inside this package: "installing" one reports it as present, an unknown one is an error
    assert install_plugin("peft") == 0
    assert install_plugin("no-such-plugin") != 0
    dest = get_benchmark_artifacts(str(tmp_path))
    assert os.path.isdir(dest) and os.listdir(dest)


# --------------------------------------------------------------------------------- class members of the GPTQ library
def test_gptq_model_wrapper_members():
    from fms_acceleration_peft.gptqmodel import GPTQModel, QuantizeConfig
    from fms_acceleration_peft.gptqmodel.models.dbrx_converted import DbrxConvertedGPTQ
    from fms_acceleration_peft.gptqmodel.nn_modules.qlinear.qlinear_tritonv2 import QuantLinear

    qc = QuantizeConfig(bits=4, group_size=32, desc_act=False, sym=True)
    m = GPTQModel.from_quantized("tiny-llama", quantize_config=qc, torch_dtype=torch.float32, device="cpu")
    assert m.device == torch.device("cpu") and m.hf_device_map is None and m.require_trust_remote_code is None
    ids = torch.randint(0, 100, (1, 4))
    out = m.generate(input_ids=ids, max_new_tokens=3)
    assert out.shape == (1, 7) and torch.equal(out[:, :4], ids)
    assert m.prepare_inputs_for_generation(ids)["input_ids"] is ids
    shards, index = m.shard_checkpoint(dict(m.model.state_dict()), max_shard_size="200KB")
    assert len(shards) > 1 and set(index["weight_map"]) == set(m.model.state_dict())
    m.warmup_triton()
    assert QuantLinear.warmup(m.model) >= 1
    assert m.fast_loss is m.model.fast_loss  # unknown attributes are looked up on the wrapped model
    with pytest.raises(AttributeError):
        m.no_such_attribute  # noqa: B018
    with pytest.raises(ValueError, match="trust_remote_code"):
        DbrxConvertedGPTQ.from_quantized("anything", quantize_config=qc)


def test_lora_parameter_tuples_have_the_reference_arity():
    from fms_acceleration_foak.fused_ops.unsloth_lora.gptq.fast_lora import GPTQuantState, extract_gptq_state
    from fms_acceleration_foak.fused_ops.unsloth_lora.gptq.fast_lora import get_lora_parameters as gptq_params
    from fms_acceleration_foak.fused_ops.unsloth_lora.utils import get_lora_parameters as dense_params
    from fms_acceleration_b200.nn.gptq import QuantLinear
    from fms_acceleration_b200.nn.lora import LoraLinear

    q = QuantLinear.random(64, 32, group_size=32, dtype=torch.float32)
    st = extract_gptq_state(q)
    assert isinstance(st, GPTQuantState) and (st.infeatures, st.outfeatures, st.group_size, st.maxq) == (64, 32, 32, 15)
    assert st.bias is None and st.trainable and not st.autogptq_cuda_available
    bare = gptq_params(q)
    assert len(bare) == 6 and bare[0].qweight is q.qweight and all(v is None for v in bare[2:])
    wrapped = LoraLinear(q, r=4, lora_alpha=8)
    qs, bias, A, B, s, drop = gptq_params(wrapped)
    assert A.shape == (4, 64) and B.shape == (32, 4) and s == 2.0 and bias is None
    wrapped.disable_adapters = True
    assert all(v is None for v in gptq_params(wrapped)[2:])

    lin = torch.nn.Linear(8, 6)
    W, qstate, bias, A, B, s, drop = dense_params(LoraLinear(lin, r=2, lora_alpha=2))
    assert W is lin.weight and qstate is None and bias is lin.bias and A.shape == (2, 8) and s == 1.0
    assert len(dense_params(lin)) == 7 and dense_params(lin)[3] is None


def test_auto_categorizer_cluster_options():
    from fms_acceleration_odm.odm.auto_categorizer import AutoCategorizeConfig, DatasetAutoCategorizer

    cfg = AutoCategorizeConfig(cluster_kwargs={"n_init": 3}, num_categories=2)
    assert cfg.cluster_algo == "kmeans"
    rng = np.random.default_rng(0)
    emb = np.concatenate([rng.normal(0, 0.1, (10, 4)), rng.normal(5, 0.1, (10, 4))])
    labels = DatasetAutoCategorizer(cfg)._cluster(emb, 2)
    assert len(set(labels[:10])) == 1 and len(set(labels[10:])) == 1 and labels[0] != labels[10]
    with pytest.raises(ValueError, match="kmeans"):
        DatasetAutoCategorizer(AutoCategorizeConfig(cluster_algo="dbscan"))._cluster(emb, 2)


def test_cli_verbs(capsys):
    from fms_acceleration.cli import cli

    assert cli(["install", "-e", "plugins/accelerated-peft", "--no-deps"]) == 0
    assert "ignored installer flags: -e --no-deps" in capsys.readouterr().out
    assert cli(["install", "no-such-plugin"]) != 0
    assert cli(["plugins"]) == 0 and "accelerated-moe" in capsys.readouterr().out
    assert cli(["configs"]) == 0 and "accelerated-peft-bnb" in capsys.readouterr().out
    assert cli(["arguments", "accelerated-peft-bnb"]) == 0
    text = capsys.readouterr().out
    # the arguments that select the configuration, then the scenarios that use it with their trainer arguments
    assert "--acceleration_framework_config_file" in text and "scenario: accelerated-peft-bnb" in text
    assert "--peft_method lora" in text and "model_name_or_path" not in text.split("arguments:")[1]
    assert cli(["arguments", "no-such-config"]) == 1


def test_apply_lora_entry_points_equal_the_unfused_projections():
    """``apply_lora_qkv / _o / _mlp_*`` of the bnb flavour on modules whose projections are LoRA over NF4 layers with
    biases: each fused call equals the projections applied one by one."""
    from fms_acceleration_foak.fused_ops.unsloth_lora.bnb.fast_lora import (apply_lora_mlp_geglu_approx,
                                                                           apply_lora_mlp_geglu_exact,
                                                                           apply_lora_mlp_swiglu, apply_lora_o,
                                                                           apply_lora_qkv)
    from fms_acceleration_b200.nn import Linear4bit
    from fms_acceleration_b200.nn.lora import LoraLinear

    torch.manual_seed(0)

    def proj(i, o):
        layer = LoraLinear(Linear4bit.from_linear(torch.nn.Linear(i, o, bias=True), "nf4", 64, torch.float32), r=4,
                           lora_alpha=8)
        torch.nn.init.normal_(layer.lora_B["default"].weight, std=0.1)
        return layer

    attn, mlp = torch.nn.Module(), torch.nn.Module()
    attn.q_proj, attn.k_proj, attn.v_proj, attn.o_proj = proj(64, 64), proj(64, 32), proj(64, 32), proj(64, 64)
    mlp.gate_proj, mlp.up_proj, mlp.down_proj = proj(64, 128), proj(64, 128), proj(128, 64)
    x = torch.randn(2, 5, 64)
    q, k, v = apply_lora_qkv(attn, x)
    for got, layer in ((q, attn.q_proj), (k, attn.k_proj), (v, attn.v_proj), (apply_lora_o(attn, x), attn.o_proj)):
        assert torch.allclose(got, layer(x), atol=1e-5)
    F = torch.nn.functional
    acts = [(apply_lora_mlp_swiglu, F.silu), (apply_lora_mlp_geglu_exact, F.gelu),
            (apply_lora_mlp_geglu_approx, lambda t: F.gelu(t, approximate="tanh"))]
    for fused, act in acts:
        want = mlp.down_proj(act(mlp.gate_proj(x)) * mlp.up_proj(x))
        assert torch.allclose(fused(mlp, x), want, atol=1e-5)
