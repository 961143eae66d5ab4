"""Worker of test_checkpoint_resume_cpu: a full state dict held by rank 0 only reaches every rank, replicated
parameters whole and expert-parallel parameters as each rank's slice; expert tensors of a checkpoint that holds all
experts are cut to the rank's share."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


class Block(torch.nn.Module):
    def __init__(self, moe):
        super().__init__()
        self.norm = torch.nn.LayerNorm(8)
        self.moe = moe


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    from fms_acceleration_b200.plugins.moe.utils.checkpoint_utils import fsdp2_load_full_state_dict
    from fms_acceleration_b200.plugins.moe.utils.scattermoe import ScatterMoE
    from fms_acceleration_b200.plugins.moe.utils.scattermoe_prepare import load_experts_onto_device

    E, H, I = 2 * world, 8, 4
    torch.manual_seed(rank)  # every rank starts from different values
    moe = ScatterMoE(H, "silu", I, E, top_k=2, dtype=torch.float32, ep_group=dist.group.WORLD)
    for p in (moe.w1.weight, moe.w2.weight, moe.w3.weight):
        p._fmsb_expert_parallel, p._fmsb_ep_group = True, dist.group.WORLD
    model = Block(moe)

    full = None
    if rank == 0:
        g = torch.Generator().manual_seed(7)
        full = {"norm.weight": torch.randn(H, generator=g), "norm.bias": torch.randn(H, generator=g),
                "moe.router.weight": torch.randn(E, H, generator=g), "moe.w1.weight": torch.randn(E, H, I, generator=g),
                "moe.w2.weight": torch.randn(E, I, H, generator=g), "moe.w3.weight": torch.randn(E, H, I, generator=g)}
    fsdp2_load_full_state_dict(None, model, full)

    # every rank can rebuild what rank 0 held: same generator, same order
    g = torch.Generator().manual_seed(7)
    want = {"norm.weight": torch.randn(H, generator=g), "norm.bias": torch.randn(H, generator=g),
            "moe.router.weight": torch.randn(E, H, generator=g), "moe.w1.weight": torch.randn(E, H, I, generator=g),
            "moe.w2.weight": torch.randn(E, I, H, generator=g), "moe.w3.weight": torch.randn(E, H, I, generator=g)}
    mine = slice(rank * 2, rank * 2 + 2)
    got = dict(model.named_parameters())
    for name in ("norm.weight", "norm.bias", "moe.router.weight"):
        assert torch.equal(got[name], want[name]), name
    for name in ("moe.w1.weight", "moe.w2.weight", "moe.w3.weight"):
        assert got[name].shape[0] == 2 and torch.equal(got[name], want[name][mine]), name

    # expert tensors of a checkpoint with all E experts -> this rank's two
    torch.manual_seed(100 + rank)
    fresh = ScatterMoE(H, "silu", I, E, top_k=2, dtype=torch.float32, ep_group=dist.group.WORLD)
    load_experts_onto_device(fresh, {"router.weight": want["moe.router.weight"], "w1.weight": want["moe.w1.weight"],
                                     "w2.weight": want["moe.w2.weight"][mine]},  # already local: taken as it is
                             dist.group.WORLD, num_experts_per_device=2)
    assert torch.equal(fresh.router.weight, want["moe.router.weight"])
    assert torch.equal(fresh.w1.weight, want["moe.w1.weight"][mine])
    assert torch.equal(fresh.w2.weight, want["moe.w2.weight"][mine])
    dist.barrier()
    if rank == 0:
        print("STATE_LOADING_OK")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
