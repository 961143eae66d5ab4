"""Smallest end-to-end configuration: tiny Llama (2 layers, hidden 256) with rank-8 LoRA on q/v, five AdamW steps,
seed 0, through the framework (plugin config -> model loader -> augmentation -> trainer) on the CPU.

The loss trace is the golden: it must be bit-reproducible between two runs, decrease, leave the base weights
untouched, and equal a hand-written reference that applies the same LoRA update without the framework.
"""
import copy

import pytest
import torch

import fms_acceleration_b200.plugins  # noqa: F401  (registers the plugins)

from fms_acceleration_b200.framework.utils.test_utils import instantiate_framework
from fms_acceleration_b200.models.builder import build_model
from fms_acceleration_b200.nn.lora import LoraConfig, LoraLinear, get_peft_model
from fms_acceleration_b200.trainer import TrainArgs, Trainer, synthetic_packed_batch


def _batches(vocab, n=5):
    return [synthetic_packed_batch(vocab, 2, 64, doc_len_range=(16, 64), seed=100 + i) for i in range(n)]


def _run(seed=0):
    torch.manual_seed(seed)
    model = build_model("tiny-llama", device="cpu", dtype=torch.float32, seed=seed)
    model = get_peft_model(model, LoraConfig(r=8, lora_alpha=16, target_modules=["q_proj", "v_proj"]))
    base = {n: p.detach().clone() for n, p in model.named_parameters() if not p.requires_grad}
    tr = Trainer(model, TrainArgs(learning_rate=1e-3, padding_free=True))
    losses = tr.train(_batches(model.config.vocab_size))
    return model, base, losses


def test_five_step_trace_is_reproducible_and_decreases():
    m1, base, l1 = _run()
    _, _, l2 = _run()
    assert l1 == l2  # bit-reproducible golden
    assert len(l1) == 5 and all(torch.isfinite(torch.tensor(l1)))
    assert l1[-1] < l1[0]
    assert abs(l1[0] - torch.log(torch.tensor(float(m1.config.vocab_size))).item()) < 1.0  # random init ~ ln(V)
    for n, p in m1.named_parameters():
        if n in base:
            assert torch.equal(p, base[n]), n  # frozen weights did not move
    n_lora = [n for n, p in m1.named_parameters() if p.requires_grad]
    assert len(n_lora) == 2 * 2 * m1.config.num_hidden_layers and all("lora_" in n for n in n_lora)
    assert sum(isinstance(m, LoraLinear) for m in m1.modules()) == 2 * m1.config.num_hidden_layers


def test_trace_equals_manual_lora_training():
    """Same five steps with LoRA applied by hand on a plain copy of the model (merged weight W + s*B@A)."""
    _, _, golden = _run()
    torch.manual_seed(0)
    model = build_model("tiny-llama", device="cpu", dtype=torch.float32, seed=0)
    peft = get_peft_model(copy.deepcopy(model), LoraConfig(r=8, lora_alpha=16, target_modules=["q_proj", "v_proj"]))
    # harvest the adapter initialisation so both runs start from the same point
    adapters = {}
    for name, mod in peft.named_modules():
        if isinstance(mod, LoraLinear):
            adapters[name.split("model.layers.")[-1]] = (mod.lora_A["default"].weight.detach().clone().requires_grad_(True),
                                                         mod.lora_B["default"].weight.detach().clone().requires_grad_(True),
                                                         mod.scaling["default"] if isinstance(mod.scaling, dict) else mod.scaling)
    for p in model.parameters():
        p.requires_grad_(False)
    params = [t for a, b, _ in adapters.values() for t in (a, b)]
    opt = torch.optim.AdamW(params, lr=1e-3, weight_decay=0.0)
    originals = {}
    for key in adapters:
        li, rest = key.split(".", 1)
        lin = model.model.layers[int(li)].get_submodule(rest)
        originals[key] = (lin, lin.weight.detach().clone())
    losses = []
    for batch in _batches(model.config.vocab_size):
        for key, (lin, w0) in originals.items():
            a, b, s = adapters[key]
            del lin._parameters["weight"]
            lin.weight = w0 + s * (b @ a)
        out = model(input_ids=batch["input_ids"], labels=batch["labels"], cu_seqlens=batch["cu_seqlens"])
        out.loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)
        losses.append(float(out.loss.detach()))
        for key, (lin, w0) in originals.items():
            del lin.weight
            lin._parameters["weight"] = torch.nn.Parameter(w0, requires_grad=False)
    assert torch.allclose(torch.tensor(losses), torch.tensor(golden), rtol=2e-4, atol=2e-4)


def test_through_the_framework_with_lora_plugin_config():
    """The accelerated-peft plugin path on the CPU is exercised up to the point that needs a GPU: configuration
    parsing, plugin activation and the requirement flags."""
    cfg = {"peft": {"quantization": {"bitsandbytes": {"quant_type": "nf4", "no_peft_model": False}}}}
    with instantiate_framework(cfg, require_packages_check=False) as fw:
        assert fw.requires_custom_loading and fw.requires_augmentation
        assert [n for n, _ in fw.active_plugins] == ["BNBAccelerationPlugin"]


@pytest.mark.parametrize("which", ["bitsandbytes", "auto_gptq"])
def test_quantised_lora_lifecycle_on_the_cpu(which):
    """Loader plugin -> augmentation -> one forward/backward with the PyTorch oracle paths: the base is quantised and
    frozen, the adapters on the targeted projections are the only trainable parameters and all of them receive a
    gradient; the consumed ``peft_config`` comes back as None."""
    from fms_acceleration_b200.nn import LoraConfig
    from fms_acceleration_b200.trainer import TrainArgs

    if which == "bitsandbytes":
        cfg = {"peft": {"quantization": {"bitsandbytes": {"quant_type": "nf4", "no_peft_model": False}}}}
        dtype, layer_cls, args = torch.bfloat16, "Linear4bit", TrainArgs(bf16=True)
    else:
        cfg = {"peft": {"quantization": {"auto_gptq": {"kernel": "triton_v2", "from_quantized": True}}}}
        dtype, layer_cls, args = torch.float16, "QuantLinear", TrainArgs(fp16=True)
    with instantiate_framework(cfg, require_packages_check=False) as fw:
        model = fw.model_loader("tiny-llama", torch_dtype=dtype, device="cpu")
        n_quant = sum(1 for m in model.modules() if m.__class__.__name__ == layer_cls)
        assert n_quant == 7 * model.config.num_hidden_layers        # q, k, v, o, gate, up, down of every layer
        peft_config = LoraConfig(r=4, lora_alpha=8, target_modules=["q_proj", "v_proj"])
        model, (returned,) = fw.augmentation(model, args, modifiable_args=(peft_config,))
        assert returned is None
    trainable = [(n, p) for n, p in model.named_parameters() if p.requires_grad]
    assert trainable and all("lora_" in n for n, _ in trainable)
    assert len(trainable) == 2 * 2 * model.config.num_hidden_layers  # A and B of q_proj and v_proj per layer
    ids = torch.randint(0, 512, (2, 16))
    out = model(input_ids=ids, labels=ids)
    out.loss.backward()
    assert torch.isfinite(out.loss.detach())
    assert all(p.grad is not None for _, p in trainable)
    # lora_B starts at zero, so only it sees a gradient on the first step; lora_A follows once B has moved
    assert any(p.grad.abs().sum() > 0 for n, p in trainable if "lora_B" in n)
