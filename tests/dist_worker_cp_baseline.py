"""Worker of test_cp_baseline_cpu: the context-parallel Mamba2 scan stated with library collectives on gloo ranks.
Every rank scans its slice from a zero state, the (final state, log total decay) pairs are all-gathered, the prefix
is combined locally and the entering-state correction added; the conv input halo comes from the previous rank.  The
result has to equal the scan (and the conv) of the whole sequence."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    from fms_acceleration_b200.ops import mamba as MB
    from fms_acceleration_b200.parallel.context_parallel import prefix_state

    torch.manual_seed(0)                                   # the same full sequence on every rank
    per, nh, P, G, N, Cc = 24, 4, 8, 2, 16, 16
    T = per * world
    x = torch.randn(T, nh, P, dtype=torch.float64)
    dt = torch.rand(T, nh, dtype=torch.float64) * 0.1 + 0.01
    A = -(torch.rand(nh, dtype=torch.float64) + 0.5)
    B = torch.randn(T, G, N, dtype=torch.float64)
    C = torch.randn(T, G, N, dtype=torch.float64)
    D = torch.randn(nh, dtype=torch.float64)
    y_full, h_full = MB.ssd_ref(x, dt, A, B, C, D, None)
    sl = slice(rank * per, (rank + 1) * per)
    y0, F_local = MB.ssd_ref(x[sl], dt[sl], A, B[sl], C[sl], D, None)
    logP = (dt[sl] * A[None, :]).sum(0)
    Fs = [torch.empty_like(F_local) for _ in range(world)]
    lPs = [torch.empty_like(logP) for _ in range(world)]
    dist.all_gather(Fs, F_local.contiguous())
    dist.all_gather(lPs, logP.contiguous())
    Fs, lPs = torch.stack(Fs), torch.stack(lPs)
    h_in = prefix_state(Fs, lPs, rank).double() if rank > 0 else torch.zeros_like(F_local)
    y = MB.state_correction_ref(y0, h_in, dt[sl], A, C[sl]).double()
    assert torch.allclose(y, y_full[sl], rtol=1e-5, atol=1e-5), (y - y_full[sl]).abs().max()
    if rank == world - 1:                                  # the last rank's leaving state is the sequence's final state
        h_out = torch.exp(lPs[rank])[:, None, None] * h_in + Fs[rank]
        assert torch.allclose(h_out.double(), h_full, rtol=1e-5, atol=1e-5)
    # conv halo: the last three input rows of the previous rank
    xc = torch.randn(T, Cc)
    w, b = torch.randn(Cc, 4) * 0.5, torch.randn(Cc)
    full = MB.conv1d_ref(xc, w, b)
    tails = [torch.empty(3, Cc) for _ in range(world)]
    dist.all_gather(tails, xc[sl][-3:].contiguous())
    halo = tails[rank - 1] if rank > 0 else None
    mine = MB.conv1d_ref(xc[sl], w, b, halo)
    assert torch.allclose(mine, full[sl], atol=1e-5)
    dist.barrier()
    if rank == 0:
        print("CP_BASELINE_OK")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
