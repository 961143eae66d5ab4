"""End-to-end parity of the fused packed path against the eager fp32 model (same quantised weights)."""
import copy

import pytest
import torch

pytestmark = pytest.mark.gpu

from fms_acceleration_b200 import _native as NV
from fms_acceleration_b200.models.builder import build_model, quantize_linears_
from fms_acceleration_b200.models.config import DecoderConfig
from fms_acceleration_b200.nn import Linear4bit, LoraConfig, get_peft_model
from fms_acceleration_b200.nn.gptq import QuantLinear
from fms_acceleration_b200.trainer import synthetic_packed_batch, to_device


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp(min=1e-12)).item()


def _cfg(d=128, **kw):
    return DecoderConfig(vocab_size=2048, hidden_size=512, intermediate_size=1024, num_hidden_layers=2,
                         num_attention_heads=512 // d, num_key_value_heads=max(512 // d // 2, 1), head_dim=d,
                         rope_theta=1e4, initializer_range=0.05, **kw)


def _float_copy(model_q):
    """fp32 CPU copy of a quantised+LoRA model with the dequantised weights as plain linears."""
    m = copy.deepcopy(model_q)

    def swap(mod):
        for name, child in list(mod.named_children()):
            if isinstance(child, Linear4bit):
                lin = torch.nn.Linear(child.in_features, child.out_features, bias=False)
                lin.weight.data = child.dequantize(dtype=torch.bfloat16).float().cpu()
                setattr(mod, name, lin)
            elif isinstance(child, QuantLinear):
                lin = torch.nn.Linear(child.infeatures, child.outfeatures, bias=False)
                lin.weight.data = child.dequantize().float().t().contiguous().cpu()
                setattr(mod, name, lin)
            else:
                swap(child)

    swap(m)
    m = m.float().cpu()
    base = m.get_base_model() if hasattr(m, "get_base_model") else m
    base.model.fused = False
    base.fast_loss = False
    base.model._rope = None
    return m


@pytest.mark.parametrize("quant,d", [("nf4", 128), ("nf4", 64), ("gptq", 128), ("none", 128)])
def test_fused_path_matches_eager(quant, d):
    torch.manual_seed(0)
    dev = torch.device("cuda")
    dtype = torch.bfloat16
    hook = None
    if quant == "nf4":
        hook = lambda layer: quantize_linears_(layer, lambda lin: Linear4bit.from_linear(lin, "nf4", 64, dtype))  # noqa: E731
    elif quant == "gptq":
        def hook(layer):
            def mk(lin):
                q = QuantLinear.random(lin.in_features, lin.out_features, 4, 128, dtype, lin.weight.device, scale_std=0.01)
                return q
            return quantize_linears_(layer, mk)
    model = build_model(_cfg(d), device=dev, dtype=dtype, layer_hook=hook)
    if quant != "none":
        model = get_peft_model(model, LoraConfig(r=16, lora_alpha=32, target_modules=["q_proj", "k_proj", "v_proj", "o_proj", "down_proj"]))
        for n, p in model.named_parameters():
            if "lora_B" in n:
                torch.nn.init.normal_(p, std=0.05)
    ref = _float_copy(model)
    base = model.get_base_model() if hasattr(model, "get_base_model") else model
    base.enable_fused("fused_ce_liger")
    batch = synthetic_packed_batch(2048, 2, 384, (16, 384), seed=3, pin=False)
    out = model(**{k: v for k, v in to_device(batch, dev).items() if k != "cu_seqlens"})
    out.loss.backward()
    NV.check_status()
    ref_out = ref(**{k: v for k, v in batch.items() if k != "cu_seqlens"})
    ref_out.loss.backward()
    assert abs(out.loss.item() - ref_out.loss.item()) < 3e-2 * max(1.0, abs(ref_out.loss.item()))
    ref_grads = {n: p.grad for n, p in ref.named_parameters() if p.grad is not None}
    checked = 0
    for n, p in model.named_parameters():
        if p.grad is None:
            continue
        assert n in ref_grads, n
        if ref_grads[n].norm() < 1e-8:
            continue
        assert _rel(p.grad.cpu(), ref_grads[n]) < 8e-2, (n, _rel(p.grad.cpu(), ref_grads[n]))
        checked += 1
    assert checked > 4
    # cu_seqlens form of the same batch gives the same loss
    out2 = model(input_ids=batch["input_ids"].to(dev), labels=batch["labels"].to(dev), cu_seqlens=batch["cu_seqlens"].to(dev))
    assert abs(out2.loss.item() - out.loss.item()) < 1e-3


def test_fused_lora_dropout_matches_masked_reference():
    """LoRA dropout in the fused projection group: forward and all gradients equal an fp32 reference that applies
    the SAME keep mask to the adapter branch only."""
    from fms_acceleration_b200.nn.lora import LoraLinear
    from fms_acceleration_b200.ops.proj import ProjGroup

    torch.manual_seed(0)
    dev = "cuda"
    T, H, O, r, p = 256, 512, 384, 16, 0.25
    lin = torch.nn.Linear(H, O, bias=False, device=dev, dtype=torch.bfloat16)
    lin.weight.requires_grad_(False)
    q = Linear4bit.from_linear(lin, "nf4", 64, torch.bfloat16)
    lora = LoraLinear(q, r, 16, lora_dropout=p).to(dev)
    with torch.no_grad():
        lora.lora_B["default"].weight.normal_(0, 0.05)  # B starts at zero: make the adapter branch visible
    lora.train()
    grp = ProjGroup([lora], "t")
    assert grp.dropout_p() == p
    x = (torch.randn(T, H, device=dev) * 0.5).bfloat16()
    dy = (torch.randn(T, O, device=dev) * 0.1).bfloat16()
    aux = {}
    y, xa = grp.forward(x, aux=aux)
    dx, grads = grp.backward(dy, x, xa, aux=aux)
    NV.check_status()
    mask, ks = aux["mask"], aux["keep_scale"]
    assert 0.6 < mask.float().mean() < 0.9 and abs(ks - 1 / (1 - p)) < 1e-6
    W = q.dequantize(dtype=torch.bfloat16).float()
    A = lora.lora_A["default"].weight.detach().float().requires_grad_()
    B = lora.lora_B["default"].weight.detach().float().requires_grad_()
    s = lora.scaling["default"]
    xr = x.float().requires_grad_()
    yr = xr @ W.t() + s * ((xr * mask * ks) @ A.t()) @ B.t()
    yr.backward(dy.float())

    def rel(a, b):
        return ((a.float() - b.float()).norm() / b.float().norm().clamp(min=1e-9)).item()

    assert rel(y, yr) < 2e-2
    assert rel(dx, xr.grad) < 3e-2
    assert rel(grads[0], A.grad) < 3e-2 and rel(grads[1], B.grad) < 3e-2
    lora.eval()
    assert grp.dropout_p() == 0.0


def test_hf_llama_uses_the_in_tree_attention_on_packed_rows():
    """A transformers Llama pointed at the registered in-tree attention: a packed row with position ids restarting
    per document gives, per document, the logits of the eager model on that document alone."""
    transformers = pytest.importorskip("transformers")
    from fms_acceleration_b200.plugins.aadp.flash_attn import HF_ATTENTION_NAME, use_in_tree_attention

    cfg = transformers.LlamaConfig(vocab_size=512, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                                   num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=1024,
                                   tie_word_embeddings=False)
    torch.manual_seed(0)
    model = transformers.LlamaForCausalLM(cfg).to("cuda", torch.bfloat16).eval()
    ref = copy.deepcopy(model)
    ref.config._attn_implementation = "eager"
    assert use_in_tree_attention(model) and model.config._attn_implementation == HF_ATTENTION_NAME
    lens = [130, 41, 129]
    docs = [torch.randint(0, 512, (1, n), device="cuda") for n in lens]
    with torch.no_grad():
        want = torch.cat([ref(input_ids=d).logits[0] for d in docs], 0).float()
        ids = torch.cat(docs, 1)
        pos = torch.cat([torch.arange(n, device="cuda") for n in lens])[None]
        got = model(input_ids=ids, position_ids=pos).logits[0].float()
    NV.check_status()
    assert ((got - want).norm() / want.norm()).item() < 3e-2
