"""Worker of test_cp_baseline_cpu: a whole Mamba2 model (and a hybrid Mamba / attention / MoE model) under the
context-parallel plugin with the library backend on gloo ranks.  Every rank holds one slice of one sequence; the sum
of the ranks' losses and of their parameter gradients has to equal the single-process model on the whole sequence."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def check(preset: str, rank: int, world: int) -> float:
    from fms_acceleration_b200.models.builder import build_model
    from fms_acceleration_b200.plugins.mcp.utils import patch_mamba_layers_with_cp_head

    per = 24
    T = per * world
    torch.manual_seed(0)
    ref = build_model(preset, device="cpu", dtype=torch.float64, seed=0)
    ids = torch.randint(0, ref.config.vocab_size, (1, T))
    ref_loss = ref(ids, labels=ids).loss
    ref_loss.backward()
    want = {n: p.grad.clone() for n, p in ref.named_parameters() if p.grad is not None}

    model = build_model(preset, device="cpu", dtype=torch.float64, seed=0)
    patch_mamba_layers_with_cp_head(model, None, rank, cp_degree=world, world_size=world)
    sl = slice(rank * per, (rank + 1) * per)
    loss = model(ids[:, sl], labels=ids[:, sl]).loss      # this slice's token losses over the global token count
    loss.backward()
    total = loss.detach().clone()
    dist.all_reduce(total)
    assert torch.allclose(total, ref_loss.detach(), atol=1e-6), (float(total), float(ref_loss))
    worst = 0.0
    for n, p in model.named_parameters():
        g = p.grad.clone() if p.grad is not None else torch.zeros_like(p)
        dist.all_reduce(g)
        if n not in want:
            assert float(g.abs().max()) == 0.0, n
            continue
        err = float((g - want[n]).abs().max())
        worst = max(worst, err)
        assert err < 1e-6, (preset, n, err)  # the state hand-off is combined in fp32
    return worst


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    os.environ.pop("FMSB_CP_BACKEND", None)  # on a CPU the library backend is the default
    worst = [check(p, rank, world) for p in ("tiny-mamba2", "tiny-granitemoehybrid")]
    dist.barrier()
    if rank == 0:
        print(f"CP_MODEL_OK worst gradient difference {max(worst):.2e}")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
