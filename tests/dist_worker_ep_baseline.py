"""Worker of test_ep_baseline_cpu: expert parallelism with library collectives on gloo ranks against the dense
oracle."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    from fms_acceleration_b200.ops.moe import moe_ref
    from fms_acceleration_b200.plugins.moe.utils.scattermoe_utils import (all_to_all_gather_inputs,
                                                                         scatter_with_routing_weights)

    torch.manual_seed(0)                       # same weights on every rank
    E, k, H, I, T = 4 * world, 2, 16, 24, 10 + rank
    router = torch.randn(E, H) * 0.5
    w1, w3, w2 = torch.randn(E, H, I) * 0.2, torch.randn(E, H, I) * 0.2, torch.randn(E, I, H) * 0.2
    torch.manual_seed(100 + rank)              # different tokens per rank
    x = torch.randn(T, H, requires_grad=True)
    logits = x.detach() @ router.t()
    wts, idx = torch.softmax(logits, -1).topk(k, -1)
    wts = wts / wts.sum(-1, keepdim=True)
    epr = E // world
    mine = slice(rank * epr, (rank + 1) * epr)
    rows, local_e, state = all_to_all_gather_inputs(x, idx, dist.group.WORLD, k, epr)
    out_rows = torch.zeros(rows.shape[0], H)
    for e in range(epr):
        sel = local_e == e
        h = torch.nn.functional.silu(rows[sel] @ w1[mine][e]) * (rows[sel] @ w3[mine][e])
        out_rows = out_rows.index_put((torch.nonzero(sel).reshape(-1),), h @ w2[mine][e])
    y = scatter_with_routing_weights(out_rows, wts, state)
    # dense statement with the same (detached) routing weights
    ref_x = x.detach().clone().requires_grad_()
    ref = torch.zeros(T, H)
    for e in range(E):
        tok, slot = torch.nonzero(idx == e, as_tuple=True)
        if tok.numel():
            h = torch.nn.functional.silu(ref_x[tok] @ w1[e]) * (ref_x[tok] @ w3[e])
            ref = ref.index_add(0, tok, (h @ w2[e]) * wts[tok, slot][:, None])
    assert torch.allclose(y, ref, atol=1e-4), (y - ref).abs().max()
    dense, _ = moe_ref(x.detach(), router, w1, w2, w3, k, idx=idx)
    assert torch.allclose(y, dense, atol=1e-4)
    g = torch.randn_like(y)
    (y * g).sum().backward()
    (ref * g).sum().backward()
    assert torch.allclose(x.grad, ref_x.grad, atol=1e-4), (x.grad - ref_x.grad).abs().max()
    # the differentiable variable-split all-to-all under its MegaBlocks name: rank r sends (r + d + 1) rows to rank d;
    # the backward brings every row's gradient back to where the row came from
    from fms_acceleration_b200.plugins.moe.utils.scattermoe_utils.megablocks import all_to_all

    send = [rank + d + 1 for d in range(world)]
    recv = [s + rank + 1 for s in range(world)]
    rows = torch.cat([torch.full((n, 3), float(100 * rank + d)) for d, n in enumerate(send)]).requires_grad_()
    got, handle = all_to_all(rows, recv, send, dist.group.WORLD)
    assert handle is None and got.shape == (sum(recv), 3)
    want_rows = torch.cat([torch.full((n, 3), float(100 * s + rank)) for s, n in enumerate(recv)])
    assert torch.equal(got, want_rows)
    (got * float(rank + 1)).sum().backward()  # the receiver scales by its rank + 1
    want_grad = torch.cat([torch.full((n, 3), float(d + 1)) for d, n in enumerate(send)])
    assert torch.equal(rows.grad, want_grad)
    dist.barrier()
    if rank == 0:
        print("EP_BASELINE_OK")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
