"""Context-parallel Mamba2 (scan hand-off and conv halo) stated with library collectives on gloo ranks equals the
single-sequence computation: the algorithm the peer-memory kernels implement, checked without a GPU."""
import os
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.parametrize("world", [2, 4])
def test_context_parallel_scan_equals_the_whole_sequence(world):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
           "127.0.0.1", "--master-port", str(29670 + world), os.path.join(HERE, "dist_worker_cp_baseline.py")]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=dict(os.environ, MASTER_ADDR="127.0.0.1"))
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    assert "CP_BASELINE_OK" in out.stdout


@pytest.mark.parametrize("world", [2, 3])
def test_context_parallel_attention_equals_the_whole_sequence(world):
    """Attention layers of hybrid models under context parallelism: keys and values gathered over the group, causal
    mask by global position; outputs, gradients (the key / value gradients summed over the ranks) and a whole hybrid
    decoder layer against the single-sequence computation."""
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
           "127.0.0.1", "--master-port", str(29680 + world), os.path.join(HERE, "dist_worker_cp_attention.py")]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=dict(os.environ, MASTER_ADDR="127.0.0.1"))
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    assert "CP_ATTENTION_OK" in out.stdout


@pytest.mark.parametrize("world", [2, 3])
def test_whole_models_under_the_library_backend_equal_the_single_process_model(world):
    """Mamba2 and the hybrid Mamba / attention / MoE model through the context-parallel plugin on gloo ranks: summed
    over the ranks, loss and every parameter gradient equal the model run on the whole sequence (labels cross the
    slice boundaries, the mean runs over the tokens of all ranks)."""
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
           "127.0.0.1", "--master-port", str(29700 + world), os.path.join(HERE, "dist_worker_cp_model.py")]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=900, env=env)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    assert "CP_MODEL_OK" in out.stdout
