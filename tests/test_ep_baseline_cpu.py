"""The library-collective statement of expert parallelism (dispatch, local experts, combine) on gloo ranks: forward
and input gradient equal the dense oracle.  Ranks hold different numbers of tokens."""
import os
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.parametrize("world", [2, 3])
def test_all_to_all_expert_parallel_matches_the_dense_oracle(world):
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
           "127.0.0.1", "--master-port", str(29650 + world), os.path.join(HERE, "dist_worker_ep_baseline.py")]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    assert "EP_BASELINE_OK" in out.stdout
