"""Multi-GPU tests: run ``tests/dist_worker.py`` under torchrun on 2 GPUs and, where the machine has them, on 4 and
8 (skipped with fewer).  NVLS is switched off for NCCL (it only bootstraps and provides the reference results
here)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


def _run(which: str, nproc: int = 2, timeout: int = 600):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", "29533", os.path.join(HERE, "dist_worker.py"), which]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=timeout)
    return res


@pytest.mark.parametrize("nproc", [2, 4, 8])
@pytest.mark.parametrize("which,expected", [
    ("comm", ["allgather", "allreduce", "reduce_scatter"]),
    ("engine", ["engine", "engine_train"]),
    ("zero1", ["zero1"]),
    ("moe", ["moe_ep", "moe_library", "moe_lora"]),
    ("cp", ["mamba_cp"]),
])
def test_multi_gpu(which, expected, nproc):
    if torch.cuda.device_count() < nproc:
        pytest.skip(f"needs {nproc} GPUs")
    res = _run(which, nproc=nproc)
    out = res.stdout + res.stderr
    assert res.returncode == 0, out[-3000:]
    for name in expected:
        assert out.count(f"DIST_OK {name}") >= nproc, f"{name} did not pass on all {nproc} ranks\n{out[-3000:]}"
