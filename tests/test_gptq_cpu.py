"""GPTQ library on the host: quantiser, Hessian solver, packing, save / load round trip, config handling."""
import json
import os

import pytest
import torch

from fms_acceleration_b200.nn.gptq import QuantLinear
from fms_acceleration_b200.ops import quant as Q
from fms_acceleration_b200.plugins.peft.gptqmodel import GPTQModel, QuantizeConfig
from fms_acceleration_b200.plugins.peft.gptqmodel.quantization.config import FORMAT
from fms_acceleration_b200.plugins.peft.gptqmodel.quantization.gptq import GPTQ
from fms_acceleration_b200.plugins.peft.gptqmodel.quantization.quantizer import Quantizer
from fms_acceleration_b200.plugins.peft.gptqmodel.utils.model import (convert_gptq_v1_to_v2_format,
                                                                      convert_gptq_v2_to_v1_format, parse_size,
                                                                      shard_checkpoint)


@pytest.mark.parametrize("bits", [2, 4, 8])
def test_pack_unpack_roundtrip(bits):
    g = torch.Generator().manual_seed(bits)
    q = torch.randint(0, 2 ** bits, (64, 32), generator=g)
    packed = Q.gptq_pack(q, bits)
    assert packed.dtype == torch.int32 and packed.shape == (64 * bits // 32, 32)
    assert torch.equal(Q.gptq_unpack(packed, bits), q)
    z = torch.randint(0, 2 ** bits, (4, 32), generator=g)
    assert torch.equal(Q.gptq_unpack_zeros(Q.gptq_pack_zeros(z, bits), bits), z)


def test_quantizer_grid():
    w = torch.randn(16, 64)
    qz = Quantizer()
    qz.configure(4, perchannel=True, sym=False)
    qz.find_params(w, weight=True)
    dq = qz.quantize(w)
    assert qz.scale.shape == (16, 1) and (dq - w).abs().max() <= qz.scale.max() * 0.5001
    levels = torch.round(dq / qz.scale + qz.zero)
    assert levels.min() >= 0 and levels.max() <= 15


def test_gptq_solver_beats_round_to_nearest():
    torch.manual_seed(0)
    lin = torch.nn.Linear(128, 48, bias=False)
    basis = torch.randn(128, 128)
    x = torch.randn(2048, 128) @ (basis * torch.logspace(0, -2, 128))  # correlated inputs
    ref = lin(x)
    W0 = lin.weight.data.clone()
    rtn = Quantizer()
    rtn.configure(4, perchannel=True, sym=True)
    g = GPTQ(lin)
    g.quantizer.configure(4, perchannel=True, sym=True)
    g.add_batch(x, ref)
    scale, zero, g_idx, *_ = g.fasterquant(percdamp=0.01, group_size=32, actorder=False)
    err_gptq = (lin(x) - ref).pow(2).mean()
    # round-to-nearest with the same group size
    Wr = torch.empty_like(W0)
    for s in range(0, 128, 32):
        rtn.find_params(W0[:, s:s + 32], weight=True)
        Wr[:, s:s + 32] = rtn.quantize(W0[:, s:s + 32])
    err_rtn = (x @ Wr.t() - ref).pow(2).mean()
    assert err_gptq < 0.8 * err_rtn
    assert scale.shape == (48, 4) and zero.shape == (48, 4) and g_idx.shape == (128,)
    # the solver's weights lie on the grid it reports, so QuantLinear.pack reproduces them exactly
    ql = QuantLinear(4, 32, 128, 48, dtype=torch.float32)
    ql.pack(lin, scale, zero, g_idx)
    assert torch.allclose(ql.dequantize().t(), lin.weight.data, atol=1e-5)


@pytest.mark.parametrize("actorder,static_groups,group_size", [(True, False, 32), (True, True, 32), (False, True, 32),
                                                               (False, False, -1), (True, False, -1)])
def test_gptq_solver_options_against_the_dense_objective(actorder, static_groups, group_size):
    """Independent oracle: the quantity GPTQ minimises is tr((W - Q) H (W - Q)^T).  Under every option the solver
    must do better on it than rounding every weight to the nearest level of the same kind of grid, and its output
    must lie on the grid it reports (scale, zero, g_idx reproduce it exactly)."""
    from fms_acceleration_b200.plugins.peft.gptqmodel.quantization.quantizer import quantize

    torch.manual_seed(1)
    cin, cout = 96, 40
    lin = torch.nn.Linear(cin, cout, bias=False)
    x = torch.randn(1024, cin) @ (torch.randn(cin, cin) * torch.logspace(0, -1.5, cin))
    x[:, 7] = 0  # an input feature that never fires
    W0 = lin.weight.data.clone()
    H = 2.0 / x.shape[0] * x.t() @ x
    g = GPTQ(lin)
    g.quantizer.configure(4, perchannel=True, sym=True)
    g.add_batch(x)
    scale, zero, g_idx, _, avg_loss = g.fasterquant(blocksize=32, percdamp=0.01, group_size=group_size,
                                                    actorder=actorder, static_groups=static_groups)
    Qw = lin.weight.data
    gs = group_size if group_size > 0 else cin
    assert scale.shape == (cout, -(-cin // gs)) and g_idx.shape == (cin,)
    # on the reported grid
    s_col, z_col = scale[:, g_idx.long()], zero[:, g_idx.long()]
    assert torch.allclose(quantize(Qw, s_col, z_col, 15), Qw, atol=1e-5)
    # better than round-to-nearest on the layer objective
    rtn = Quantizer()
    rtn.configure(4, perchannel=True, sym=True)
    Wr = torch.empty_like(W0)
    for c in range(0, cin, gs):
        rtn.find_params(W0[:, c:c + gs], weight=True)
        Wr[:, c:c + gs] = rtn.quantize(W0[:, c:c + gs])

    def objective(Wq):
        d = (W0 - Wq)
        d[:, 7] = 0  # the silent feature does not enter the objective
        return torch.trace(d @ H @ d.t()).item()

    assert objective(Qw) < 0.9 * objective(Wr), (objective(Qw), objective(Wr))
    assert avg_loss >= 0


def test_clipping_search_matches_a_plain_loop():
    """The vectorised search over shrink factors picks, per row, the first factor with the smallest error."""
    from fms_acceleration_b200.plugins.peft.gptqmodel.quantization.quantizer import quantize

    torch.manual_seed(2)
    w = torch.randn(12, 50) * torch.logspace(0, 1, 12)[:, None]
    w[3, 10] = 40.0  # an outlier that a tighter range should clip
    for sym in (True, False):
        qz = Quantizer()
        qz.configure(3, perchannel=True, sym=sym, mse=True, norm=2.4, grid=50, maxshrink=0.8)
        qz.find_params(w, weight=True)
        plain = Quantizer()
        plain.configure(3, perchannel=True, sym=sym)
        plain.find_params(w, weight=True)
        lo = torch.minimum(w.amin(1), torch.zeros(12))
        hi = torch.maximum(w.amax(1), torch.zeros(12))
        if sym:
            b = torch.maximum(lo.abs(), hi)
            lo, hi = torch.where(lo < 0, -b, lo), b
        for r in range(12):
            best, arg = float("inf"), None
            for i in range(int(0.8 * 50)):
                f = 1 - i / 50
                sc = f * (hi[r] - lo[r]) / 7
                zp = plain.zero[r, 0] if sym else torch.round(-f * lo[r] / sc)
                e = (quantize(w[r], sc, zp, 7) - w[r]).abs().pow(2.4).sum().item()
                if e < best:
                    best, arg = e, (sc, zp)
            assert torch.allclose(qz.scale[r, 0], arg[0], rtol=1e-5) and torch.allclose(qz.zero[r, 0], arg[1])
        assert (qz.quantize(w) - w).abs().pow(2.4).sum() <= (plain.quantize(w) - w).abs().pow(2.4).sum() + 1e-4


def test_v1_v2_zero_point_conversion():
    ql = QuantLinear.random(64, 32, 4, 32, torch.float32)
    model = torch.nn.Sequential(ql)
    before = ql.qzeros.clone()
    convert_gptq_v2_to_v1_format(model, 4)
    assert torch.equal(Q.gptq_unpack_zeros(ql.qzeros, 4), Q.gptq_unpack_zeros(before, 4) - 1)
    convert_gptq_v1_to_v2_format(model, 4)
    assert torch.equal(ql.qzeros, before)


def test_quantize_config_roundtrip(tmp_path):
    qc = QuantizeConfig(bits=4, group_size=64, desc_act=False)
    qc.save_pretrained(str(tmp_path))
    back = QuantizeConfig.from_pretrained(str(tmp_path))
    assert (back.bits, back.group_size, back.desc_act, back.sym) == (4, 64, False, True)
    legacy = QuantizeConfig.from_quant_config({"bits": 4, "group_size": 128, "is_marlin_format": False,
                                               "checkpoint_format": "gptq", "unknown_key": 1})
    assert legacy.format == FORMAT.GPTQ and legacy.group_size == 128
    with pytest.raises(ValueError):
        QuantizeConfig(bits=5)
    with pytest.raises(ValueError):
        QuantizeConfig(bits=4, group_size=-7)


def test_shard_checkpoint_and_sizes():
    assert parse_size("2GB") == 2 * 2 ** 30 and parse_size("1GiB") == 2 ** 30 and parse_size(17) == 17
    sd = {f"t{i}": torch.zeros(1000) for i in range(5)}
    shards, index = shard_checkpoint(sd, 8500, "model.safetensors")
    assert len(shards) == 3 and set(index["weight_map"]) == set(sd)
    one, idx = shard_checkpoint(sd, 10 ** 9, "model.safetensors")
    assert list(one) == ["model.safetensors"] and idx is None


def test_quantize_save_load_tiny_llama(tmp_path):
    torch.manual_seed(0)
    qc = QuantizeConfig(bits=4, group_size=32, desc_act=False)
    wrapper = GPTQModel.from_pretrained("tiny-llama", qc, torch_dtype=torch.float32)
    model = wrapper.model
    ids = torch.randint(0, model.config.vocab_size, (2, 24))
    ref_logits = model(ids).logits.detach()
    calib = [{"input_ids": torch.randint(0, model.config.vocab_size, (32,)), "attention_mask": torch.ones(32)}
             for _ in range(8)]
    wrapper.quantize(calib, batch_size=4)
    n_q = sum(isinstance(m, QuantLinear) for m in model.modules())
    assert n_q == 7 * model.config.num_hidden_layers
    q_logits = model(ids).logits.detach()
    rel = (q_logits - ref_logits).norm() / ref_logits.norm()
    assert rel < 0.5  # random-init weights at 4 bits: coarse, but far from unrelated
    out = tmp_path / "ckpt"
    wrapper.save_quantized(str(out))
    cfg = json.load(open(out / "config.json"))
    assert cfg["quantization_config"]["bits"] == 4 and os.path.exists(out / "quantize_config.json")
    loaded = GPTQModel.from_quantized(str(out), torch_dtype=torch.float32)
    assert loaded.quantized and torch.allclose(loaded.model(ids).logits, q_logits, atol=5e-3)  # scales are stored in fp16
    with pytest.raises(EnvironmentError):
        wrapper.quantize(calib)


def test_moe_layer_names_expand_per_expert():
    from fms_acceleration_b200.plugins.peft.gptqmodel.utils.model import EXPERT_INDEX_PLACEHOLDER, get_moe_layer_modules

    groups = [["self_attn.q_proj"], [f"moe.experts.{EXPERT_INDEX_PLACEHOLDER}.w1", "moe.gate"]]
    out = get_moe_layer_modules(groups, 3)
    assert out == [["self_attn.q_proj"], ["moe.experts.0.w1", "moe.experts.1.w1", "moe.experts.2.w1", "moe.gate"]]


def test_simple_dispatch_and_hash(tmp_path):
    from fms_acceleration_b200.plugins.peft.gptqmodel.utils.model import (find_tied_parameters, simple_dispatch_model,
                                                                         verify_file_hash)
    import hashlib

    class Tiny(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.emb = torch.nn.Embedding(8, 4)
            self.body = torch.nn.Linear(4, 4)
            self.head = torch.nn.Linear(4, 8, bias=False)
            self.head.weight = self.emb.weight

        def forward(self, ids):
            return self.head(self.body(self.emb(ids)))

    m = Tiny()
    assert find_tied_parameters(m) == [["emb.weight", "head.weight"]]
    m = simple_dispatch_model(m, {"emb": "cpu", "body": "cpu", "head": "cpu"})
    assert m.head.weight is m.emb.weight and m.hf_device_map["body"] == "cpu"
    assert m(torch.tensor([[1, 2]])).shape == (1, 2, 8)
    m2 = simple_dispatch_model(Tiny(), {"": "cpu"})
    assert m2.hf_device_map == {"": "cpu"}
    f = tmp_path / "blob.bin"
    f.write_bytes(b"abc" * 1000)
    assert verify_file_hash(str(f), "sha256:" + hashlib.sha256(b"abc" * 1000).hexdigest())
    assert not verify_file_hash(str(f), "md5:" + "0" * 32)


def test_gptq_lora_model_never_merges():
    from fms_acceleration_b200.nn.lora import LoraConfig
    from fms_acceleration_b200.plugins.peft.gptqmodel.utils.peft import (PEFT_TYPE_TO_MODEL_MAPPING, GPTQLoraLinear,
                                                                        GPTQLoraModel, get_gptq_peft_model,
                                                                        hijack_peft_mappings)

    class Block(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.q_proj = QuantLinear(4, 32, 32, 16, bias=False)
            self.lm_head = torch.nn.Linear(16, 8)

    before = PEFT_TYPE_TO_MODEL_MAPPING["LORA"]
    with hijack_peft_mappings():
        assert PEFT_TYPE_TO_MODEL_MAPPING["LORA"] is GPTQLoraModel
    assert PEFT_TYPE_TO_MODEL_MAPPING["LORA"] is before
    pm = get_gptq_peft_model(Block(), LoraConfig(r=4, lora_alpha=8, target_modules=None), auto_find_all_linears=True)
    assert isinstance(pm, GPTQLoraModel)
    assert isinstance(pm.base_model.model.q_proj, GPTQLoraLinear)
    with pytest.raises(NotImplementedError):
        pm.merge_and_unload()


def test_importer_and_reference_import_paths():
    from fms_acceleration_peft.gptqmodel.nn_modules.qlinear import BaseQuantLinear
    from fms_acceleration_peft.gptqmodel.nn_modules.qlinear.qlinear_tritonv2 import QuantLinear as TV2
    from fms_acceleration_peft.gptqmodel.nn_modules.triton_utils.dequant import dequant248, quant_matmul_248
    from fms_acceleration_peft.gptqmodel.utils.backend import Backend
    from fms_acceleration_peft.gptqmodel.utils.importer import select_quant_linear

    assert TV2 is QuantLinear and BaseQuantLinear is QuantLinear
    assert select_quant_linear(4, 128, False, True, Backend.AUTO, FORMAT.GPTQ, pack=True) is QuantLinear
    assert select_quant_linear(8, -1, True, False, Backend.TRITON, FORMAT.GPTQ_V2) is QuantLinear
    assert not QuantLinear.validate(3, 128, False, True, raise_error=False)
    with pytest.raises(NotImplementedError):
        select_quant_linear(3, 128, False, True, Backend.TRITON, FORMAT.GPTQ_V2)
    # dequantise-then-matmul helpers on the CPU oracle path
    torch.manual_seed(0)
    layer = QuantLinear(4, 32, 64, 48, dtype=torch.float32)
    lin = torch.nn.Linear(64, 48, bias=False)
    q = Quantizer()
    q.configure(4, perchannel=True, sym=True)
    groups = []
    for g in range(2):
        q.find_params(lin.weight.data[:, g * 32:(g + 1) * 32], weight=True)
        groups.append((q.scale.clone(), q.zero.clone()))
    scales = torch.cat([s for s, _ in groups], 1)
    zeros = torch.cat([z for _, z in groups], 1)
    layer.pack(lin, scales, zeros, None)
    W = dequant248(layer.qweight, layer.scales, layer.qzeros, layer.g_idx, 4, zero_offset=layer.zero_offset)
    assert W.shape == (64, 48)
    x = torch.randn(3, 64)
    if layer.zero_offset == 0:
        y = quant_matmul_248(x, layer.qweight, layer.scales, layer.qzeros, layer.g_idx, 4)
        assert torch.allclose(y, x @ W, atol=1e-5)
        yt = quant_matmul_248(torch.randn(3, 48), layer.qweight, layer.scales, layer.qzeros, layer.g_idx, 4, transpose=True)
        assert yt.shape == (3, 64)
    assert (W.t() - lin.weight.data).abs().max() < 0.2 * lin.weight.data.abs().max()
