"""Expert-parallel checks run under torchrun by tests/dist_worker.py."""
import torch
import torch.distributed as dist


def check_moe(dev, rank, world):
    from fms_acceleration_b200 import _native as NV
    from fms_acceleration_b200.ops import moe as MOE
    from fms_acceleration_b200.plugins.moe.utils.scattermoe import ScatterMoE

    T, H, I, E, k = 512, 512, 256, 8, 2
    torch.manual_seed(7)
    full = {n: torch.randn(s, device=dev) * 0.05 for n, s in
            (("router", (E, H)), ("w1", (E, H, I)), ("w2", (E, I, H)), ("w3", (E, H, I)))}
    per = E // world
    moe = ScatterMoE(H, "silu", I, E, top_k=k, dtype=torch.bfloat16, device=dev, ep_group=dist.group.WORLD)
    with torch.no_grad():
        moe.router.weight.copy_(full["router"])
        for n in ("w1", "w2", "w3"):
            getattr(moe, n).weight.copy_(full[n][rank * per: (rank + 1) * per])
    torch.manual_seed(100 + rank)
    x = (torch.randn(T, H, device=dev) * 0.5).bfloat16().requires_grad_()
    g = torch.randn(T, H, device=dev).bfloat16()
    for it in range(2):  # twice: buffers and epochs are reused
        x.grad = None
        moe.zero_grad()
        out, logits = moe(x)
        out.backward(g)
    NV.check_status()
    _, kidx = MOE.router_topk(logits.detach(), k)
    xf = x.detach().float().requires_grad_()
    ws = {n: v.bfloat16().float().requires_grad_() for n, v in full.items()}
    ref, _ = MOE.moe_ref(xf, ws["router"], ws["w1"], ws["w2"], ws["w3"], k, idx=kidx)
    ref.backward(g.float())

    def rel(a, b):
        return ((a.float() - b.float()).norm() / b.float().norm().clamp(min=1e-12)).item()

    assert rel(out, ref) < 2e-2, rel(out, ref)
    assert rel(x.grad, xf.grad) < 3e-2, rel(x.grad, xf.grad)
    # expert gradients: the owner holds the sum over the tokens of ALL ranks
    for n in ("w1", "w2", "w3"):
        gsum = ws[n].grad.clone()
        dist.all_reduce(gsum)
        mine = getattr(moe, n).weight.grad
        assert rel(mine, gsum[rank * per: (rank + 1) * per]) < 3e-2, (n, rel(mine, gsum[rank * per: (rank + 1) * per]))
    print("DIST_OK moe_ep", flush=True)
