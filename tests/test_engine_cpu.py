"""Host-side logic of the multi-rank engine on gloo ranks: gradient segments reduced from autograd hooks, gradient
accumulation, the rank-sharded optimizer and its resume, and the expert-parallel checkpoint (every rank's experts
written, converted and resumed)."""
import os
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


def _run(which, world, tmp_path, port):
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", FMSB_MOE_BACKEND="library")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
           "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "dist_worker_engine_cpu.py"), which, str(tmp_path)]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=900, env=env)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-5000:]
    return out.stdout


def test_gradient_segments_are_reduced_from_the_hooks(tmp_path):
    assert _run("reduce", 2, tmp_path, 29701).count("CPU_OK overlapped_reduce") == 2


@pytest.mark.parametrize("world", [2, 4])
def test_sharded_optimizer_matches_replicated_and_resumes(tmp_path, world):
    assert _run("zero1", world, tmp_path, 29702 + world).count("CPU_OK zero1_resume") == world


@pytest.mark.parametrize("world", [2, 4])
def test_expert_parallel_checkpoint_holds_every_rank(tmp_path, world):
    assert _run("ep_ckpt", world, tmp_path, 29712 + world).count("CPU_OK ep_checkpoint") == world


def test_expert_lora_under_expert_parallelism(tmp_path):
    assert _run("ep_lora", 2, tmp_path, 29731).count("CPU_OK ep_lora") == 2


def test_in_tree_adamw_matches_torch_on_cpu_and_shares_its_state_layout():
    """ops.optim.AdamW: same numbers as torch.optim.AdamW (fp32 parameters, CPU fall-back path) over several steps,
    and a state_dict that torch's optimizer loads (and vice versa)."""
    import torch

    from fms_acceleration_b200.ops.optim import AdamW

    torch.manual_seed(0)
    ws = [torch.randn(33, 7), torch.randn(5)]
    a = [w.clone().requires_grad_() for w in ws]
    b = [w.clone().requires_grad_() for w in ws]
    oa = AdamW(a, lr=1e-2, weight_decay=0.1)
    ob = torch.optim.AdamW(b, lr=1e-2, weight_decay=0.1)
    for it in range(4):
        gs = [torch.randn_like(w) for w in ws]
        for p, q, g in zip(a, b, gs):
            p.grad, q.grad = g.clone(), g.clone()
        oa.step()
        ob.step()
    for p, q in zip(a, b):
        assert torch.allclose(p, q, atol=1e-6, rtol=1e-5)
    sd = oa.state_dict()
    assert set(sd["state"][0]) == {"step", "exp_avg", "exp_avg_sq"} and float(sd["state"][0]["step"]) == 4.0
    ob2 = torch.optim.AdamW([w.clone().requires_grad_() for w in ws], lr=1e-2, weight_decay=0.1)
    ob2.load_state_dict(sd)
    oa2 = AdamW([w.clone().requires_grad_() for w in ws], lr=1e-2, weight_decay=0.1)
    oa2.load_state_dict(ob.state_dict())
    assert float(oa2.state_dict()["state"][1]["step"]) == 4.0
