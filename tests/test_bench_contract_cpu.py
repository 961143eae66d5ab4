"""bench.py pieces that need no GPU: configuration per benchmark and world size, synthetic batch shapes, the reference
arm's one-line answer."""
import importlib.util
import json
import os
import subprocess
import sys

import pytest

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(REPO, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_configs_name_the_published_rows():
    b = _bench()
    assert set(b.CONFIGS) == {"mistral-qlora", "granite-moe", "llama70b-gptq", "mamba-cp"}
    metric, preset, batch, seq, published = b.CONFIGS["mistral-qlora"]
    assert (preset, batch, seq, published) == ("mistral-7b", 4, 4096, 4128.0) and "Mistral-7B NF4 QLoRA" in metric
    assert b.CONFIGS["granite-moe"][1:] == ("granite-3b-a800m", 8, 2048, 6216.0)
    assert b.CONFIGS["llama70b-gptq"][4] == 496.0


@pytest.mark.parametrize("world,ep", [(1, 1), (2, 2), (4, 4), (8, 8), (3, 1), (6, 2)])
def test_expert_parallel_degree_follows_the_world_size(world, ep):
    cfg = _bench().framework_config("granite-moe", world)
    assert cfg["training"]["moe"]["scattermoe"]["ep_degree"] == ep


def test_framework_configs_use_the_reference_key_paths():
    b = _bench()
    m = b.framework_config("mistral-qlora", 1)
    assert m["peft"]["quantization"]["bitsandbytes"]["quant_type"] == "nf4"
    assert m["peft"]["quantization"]["fused_ops_and_kernels"]["base_layer"] == "bitsandbytes"
    assert m["training"]["attention"]["padding_free"]["method"] == "huggingface"
    g = b.framework_config("llama70b-gptq", 8)
    assert g["peft"]["quantization"]["auto_gptq"] == {"kernel": "triton_v2", "from_quantized": True}
    assert "mamba" not in b.framework_config("mamba-cp", 1)["training"]
    assert b.framework_config("mamba-cp", 4)["training"]["mamba"]["cp"]["degree"] == 4


def test_synthetic_batches_have_the_benchmark_shape():
    from fms_acceleration_b200.models.builder import resolve_config

    b = _bench()
    cfg = resolve_config("tiny-llama")
    batches, tokens = b.make_batches("mistral-qlora", cfg, 2, 256, rank=1, world=4, n_batches=2)
    assert tokens == 2 * 256 * 4 and len(batches) == 2
    for bt in batches:
        assert bt["input_ids"].shape == (1, 512) and bt["labels"].shape == (1, 512)
        cu = bt["cu_seqlens"]
        assert int(cu[0]) == 0 and int(cu[-1]) == 512 and (cu[1:] > cu[:-1]).all()
        assert (bt["labels"][0, cu[:-1].long()] == -100).all()  # the first token of a document is never a target
    mb, mtok = b.make_batches("mamba-cp", cfg, 1, 1024, rank=2, world=4, n_batches=1)
    assert mtok == 1024 and mb[0]["input_ids"].shape == (1, 256)


def test_reference_arm_prints_one_json_line_and_exits_zero():
    out = subprocess.run([sys.executable, os.path.join(REPO, "bench.py"), "--impl", "reference", "--gpus", "1"],
                         capture_output=True, text=True, timeout=300)
    assert out.returncode == 0
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and ("unavailable" in line or "value" in line)


def test_clock_sampler_parses_nvidia_smi_lines():
    """Median SM clock, maximum clock and the set of active throttle reasons from `nvidia-smi --format=csv` lines."""
    import tempfile

    b = _bench()

    class _Done:
        def terminate(self):
            pass

        def wait(self, timeout=None):
            return 0

        def kill(self):
            pass

    s = b.ClockSampler.__new__(b.ClockSampler)
    s.tmp = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
    s.tmp.write("0, 1965, 1965, 412.5, 0x0000000000000000, Not Active, Not Active, Not Active, Not Active\n"
                "0, 1500, 1965, 998.1, 0x0000000000000004, Not Active, Not Active, Not Active, Active\n"
                "0, 1470, 1965, 1001.0, 0x0000000000000004, Not Active, Not Active, Not Active, Active\n"
                "garbage line\n")
    s.proc = _Done()
    out = s.stop()
    assert out["sm_mhz"] == 1500.0 and out["sm_max_mhz"] == 1965.0 and out["samples"] == 3
    assert out["reasons"] == ["sw_power_cap"]
    # no sampler process (nvidia-smi missing): the keys are still there
    s2 = b.ClockSampler.__new__(b.ClockSampler)
    s2.proc, s2.tmp = None, None
    assert s2.stop() == {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
