"""The library-kernel comparison arm computes the same function as the model it wraps (CPU: torch formulations of
every piece; the reference's Triton files and flash-attn only load on a GPU)."""
import os

import pytest
import torch

from fms_acceleration_b200.baseline import BaselineRunner, reference_kernels_status
from fms_acceleration_b200.baseline import backend as BK
from fms_acceleration_b200.models.builder import build_model
from fms_acceleration_b200.nn.lora import LoraConfig, get_peft_model
from fms_acceleration_b200.trainer import synthetic_packed_batch


@pytest.mark.parametrize("name,lora", [("tiny-llama", True), ("tiny-llama", False), ("tiny-granitemoe", False)])
def test_baseline_runner_matches_the_model(name, lora):
    torch.manual_seed(0)
    model = build_model(name, dtype=torch.float32, seed=0)
    if name == "tiny-granitemoe":
        from fms_acceleration_b200.plugins.moe.utils import prepare_scattermoe

        prepare_scattermoe(model, None, 0, 1, 1)
    if lora:
        model = get_peft_model(model, LoraConfig(r=4, lora_alpha=8, target_modules=["q_proj", "v_proj"]))
        for n, p in model.named_parameters():
            if "lora_B" in n:
                torch.nn.init.normal_(p, std=0.05)
    V = (model.get_base_model() if lora else model).config.vocab_size
    b = synthetic_packed_batch(min(V, 1024), 2, 40, (8, 40), seed=3, pin=False)
    ref = model(input_ids=b["input_ids"], labels=b["labels"], cu_seqlens=b["cu_seqlens"]).loss
    ref.backward()
    want = {n: p.grad.clone() for n, p in model.named_parameters() if p.grad is not None}
    model.zero_grad()
    runner = BaselineRunner(model)
    got = runner(input_ids=b["input_ids"], labels=b["labels"], cu_seqlens=b["cu_seqlens"]).loss
    got.backward()
    assert abs(got.item() - ref.item()) < 1e-5
    for n, p in model.named_parameters():
        if n in want:
            assert torch.allclose(p.grad, want[n], atol=1e-5, rtol=1e-4), n
    assert "attention" in reference_kernels_status()


def test_reference_files_load_by_path_without_their_package_inits():
    """The loader registers every package level as an empty module, so a leaf file imports although the packages'
    own ``__init__`` files need peft / accelerate / bitsandbytes."""
    if not os.path.isdir(os.path.join(BK.REF_ROOT, "fms_acceleration_foak")):
        pytest.skip("no copy of the reference under baseline/_ref")
    pytest.importorskip("triton")
    mod = BK._load_reference("fms_acceleration_foak", "fused_ops.unsloth_lora.swiglu")
    assert hasattr(mod, "swiglu_fg_kernel") and hasattr(mod, "swiglu_DWf_DW_dfg_kernel")
    rms = BK._load_reference("fms_acceleration_foak", "kernels.unsloth.rms_layernorm")
    assert hasattr(rms, "fast_rms_layernorm")
    lce = BK._load_reference("fms_acceleration_foak", "fused_ops.liger_ce.fused_linear_cross_entropy_loss")
    assert hasattr(lce, "LigerFusedLinearCrossEntropyFunction")
