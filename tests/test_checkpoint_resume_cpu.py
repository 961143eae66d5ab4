"""Trainer checkpoints: resume reproduces the uninterrupted run; the layout is the DCP / PEFT one."""
import json
import os

import pytest
import torch

from fms_acceleration_b200.models.builder import build_model
from fms_acceleration_b200.nn.lora import LoraConfig, get_peft_model
from fms_acceleration_b200.trainer import TrainArgs, Trainer, synthetic_packed_batch


def _make(lora: bool, out: str, name="tiny-llama"):
    torch.manual_seed(0)
    model = build_model(name, dtype=torch.float32, seed=0)
    if lora:
        model = get_peft_model(model, LoraConfig(r=4, lora_alpha=8, target_modules=["q_proj", "v_proj"]))
    return Trainer(model, TrainArgs(learning_rate=1e-3, output_dir=out, save_steps=3, weight_decay=0.01))


def _batches(vocab, lo, hi):
    return [synthetic_packed_batch(vocab, 2, 48, (8, 48), seed=500 + i) for i in range(lo, hi)]


@pytest.mark.parametrize("lora", [True, False])
def test_resume_matches_uninterrupted_run(tmp_path, lora):
    out = str(tmp_path / "run")
    a = _make(lora, out)
    V = a.model.config.vocab_size
    full = a.train(_batches(V, 0, 6))
    ckpt = os.path.join(out, "checkpoint-3")
    assert Trainer.latest_checkpoint(out).endswith("checkpoint-6")
    assert os.path.isdir(os.path.join(ckpt, "pytorch_model_fsdp_0")) and os.path.isdir(os.path.join(ckpt, "optimizer_0"))
    assert json.load(open(os.path.join(ckpt, "trainer_state.json")))["global_step"] == 3
    assert os.path.exists(os.path.join(ckpt, "adapter_model.safetensors")) == lora
    b = _make(lora, str(tmp_path / "other"))
    b.args.save_steps = 0
    b.load_checkpoint(ckpt)
    assert b.global_step == 3 and len(b.log_history) == 3
    resumed = b.train(_batches(V, 3, 6))
    assert resumed == pytest.approx(full[3:], rel=1e-6, abs=1e-7)
    for (n1, p1), (n2, p2) in zip(a.model.named_parameters(), b.model.named_parameters()):
        assert torch.allclose(p1, p2, atol=1e-7), n1


def test_lora_checkpoint_holds_only_adapters(tmp_path):
    from safetensors.torch import load_file

    out = str(tmp_path / "run")
    t = _make(True, out)
    t.train(_batches(t.model.config.vocab_size, 0, 3))
    sd = load_file(os.path.join(out, "checkpoint-3", "adapter_model.safetensors"))
    assert sd and all("lora_" in k for k in sd)
    # PEFT's key layout: no adapter name between ``lora_A`` / ``lora_B`` and ``weight``
    assert all(k.endswith(("lora_A.weight", "lora_B.weight")) and k.startswith("base_model.model.") for k in sd)
    cfg = json.load(open(os.path.join(out, "checkpoint-3", "adapter_config.json")))
    assert cfg["r"] == 4 and sorted(cfg["target_modules"]) == ["q_proj", "v_proj"]


def test_truncated_shard_is_detected(tmp_path):
    """A damaged checkpoint must fail loudly on load, not resume from garbage."""
    out = str(tmp_path / "run")
    t = _make(False, out)
    t.train(_batches(t.model.config.vocab_size, 0, 3))
    shard_dir = os.path.join(out, "checkpoint-3", "pytorch_model_fsdp_0")
    shard = [f for f in os.listdir(shard_dir) if f.endswith(".distcp")][0]
    path = os.path.join(shard_dir, shard)
    size = os.path.getsize(path)
    with open(path, "r+b") as fh:
        fh.truncate(size // 3)
    fresh = _make(False, str(tmp_path / "x"))
    with pytest.raises(RuntimeError, match="incomplete or damaged"):
        fresh.load_checkpoint(os.path.join(out, "checkpoint-3"))


@pytest.mark.parametrize("world", [2, 3])
def test_full_state_dict_of_rank_zero_reaches_every_rank(world):
    """``fsdp2_load_full_state_dict`` / ``load_experts_onto_device`` on gloo ranks: replicated parameters arrive whole,
    expert-parallel ones as each rank's slice."""
    import subprocess
    import sys

    here = os.path.dirname(os.path.abspath(__file__))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
           "127.0.0.1", "--master-port", str(29670 + world), os.path.join(here, "dist_worker_state_loading.py")]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=dict(os.environ, MASTER_ADDR="127.0.0.1"))
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    assert "STATE_LOADING_OK" in out.stdout


def test_adapter_round_trip_and_merge(tmp_path):
    """``save_pretrained`` -> ``PeftModelShim.from_pretrained`` on a fresh base gives the same function; the adapter
    file of a trainer checkpoint loads the same way; ``merge_and_unload`` folds the adapters into dense weights and a
    packed base refuses the merge."""
    from fms_acceleration_b200.models.builder import quantize_linears_
    from fms_acceleration_b200.nn import Linear4bit
    from fms_acceleration_b200.nn.lora import PeftModelShim

    torch.manual_seed(0)
    model = get_peft_model(build_model("tiny-llama", seed=0), LoraConfig(r=4, lora_alpha=8, target_modules=["q_proj", "v_proj"]))
    for name, p in model.named_parameters():
        if "lora_B" in name:
            torch.nn.init.normal_(p, std=0.05)
    ids = torch.randint(0, 1000, (1, 12))
    want = model(ids, return_logits=True).logits
    model.save_pretrained(str(tmp_path / "adapter"))
    again = PeftModelShim.from_pretrained(build_model("tiny-llama", seed=0), str(tmp_path / "adapter"))
    assert torch.allclose(again(ids, return_logits=True).logits, want, atol=1e-6)
    assert not any(p.requires_grad for p in again.parameters())
    trainable = PeftModelShim.from_pretrained(build_model("tiny-llama", seed=0), str(tmp_path / "adapter"), is_trainable=True)
    assert sum(p.requires_grad for p in trainable.parameters()) == 2 * 2 * 2  # (A, B) x 2 projections x 2 layers
    plain = again.merge_and_unload()
    assert not any("lora" in n for n, _ in plain.named_parameters())
    assert torch.allclose(plain(ids, return_logits=True).logits, want, atol=1e-4)

    # the adapter file a trainer checkpoint writes
    t = _make(True, str(tmp_path / "run"))
    t.train(_batches(t.model.config.vocab_size, 0, 3))
    from_ckpt = PeftModelShim.from_pretrained(build_model("tiny-llama", seed=0), str(tmp_path / "run" / "checkpoint-3"))
    for (n1, a), (n2, b) in zip(sorted(t.model.adapter_state_dict().items()), sorted(from_ckpt.adapter_state_dict().items())):
        assert n1 == n2 and torch.equal(a, b)

    packed = build_model("tiny-llama", seed=0, layer_hook=lambda layer: quantize_linears_(
        layer, lambda lin: Linear4bit.from_linear(lin, "nf4", 64, torch.float32)))
    with pytest.raises(NotImplementedError):
        get_peft_model(packed, LoraConfig(r=4, lora_alpha=8, target_modules=["q_proj"])).merge_and_unload()
