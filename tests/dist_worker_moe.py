"""Expert-parallel checks run under torchrun by tests/dist_worker.py."""
import os

import torch
import torch.distributed as dist


def _case(dev, rank, world, T, chunks, budget, tag):
    from fms_acceleration_b200 import _native as NV
    from fms_acceleration_b200.ops import moe as MOE
    from fms_acceleration_b200.plugins.moe.utils.scattermoe import ScatterMoE

    H, I, E, k = 512, 256, 8, 2
    if E % world:
        E = 2 * world
    os.environ["FMSB_MOE_CHUNKS"] = str(chunks)
    MOE.MoEContext._shared.clear()
    torch.manual_seed(7)
    full = {n: torch.randn(s, device=dev) * 0.05 for n, s in
            (("router", (E, H)), ("w1", (E, H, I)), ("w2", (E, I, H)), ("w3", (E, H, I)))}
    per = E // world
    moe = ScatterMoE(H, "silu", I, E, top_k=k, dtype=torch.bfloat16, device=dev, ep_group=dist.group.WORLD,
                     token_budget=budget)
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
    assert MOE.overflow_count(dev, reset=True) == 0
    _, kidx = MOE.router_topk(logits.detach(), k)
    xf = x.detach().float().requires_grad_()
    ws = {n: v.bfloat16().float().requires_grad_() for n, v in full.items()}
    ref, _ = MOE.moe_ref(xf, ws["router"], ws["w1"], ws["w2"], ws["w3"], k, idx=kidx)
    ref.backward(g.float())

    def rel(a, b):
        return ((a.float() - b.float()).norm() / b.float().norm().clamp(min=1e-12)).item()

    assert rel(out, ref) < 2e-2, (tag, rel(out, ref))
    assert rel(x.grad, xf.grad) < 3e-2, (tag, rel(x.grad, xf.grad))
    # the router's gradient comes through the routing weights (4 bytes per pair read back from the owners)
    assert rel(moe.router.weight.grad, ws["router"].grad) < 8e-2, (tag, rel(moe.router.weight.grad, ws["router"].grad))
    # expert gradients: the owner holds the sum over the tokens of ALL ranks
    for n in ("w1", "w2", "w3"):
        gsum = ws[n].grad.clone()
        dist.all_reduce(gsum)
        mine = getattr(moe, n).weight.grad
        assert rel(mine, gsum[rank * per: (rank + 1) * per]) < 3e-2, (tag, n, rel(mine, gsum[rank * per: (rank + 1) * per]))


def check_moe(dev, rank, world):
    # equal token counts, two chunks (the default)
    _case(dev, rank, world, 512, 2, 512, "equal")
    # ranks bring different numbers of tokens (padding-free batches), below the agreed budget; three chunks, so the
    # two staging sets are reused inside one call
    _case(dev, rank, world, 512 - 56 * rank, 3, 640, "unequal")
    # one chunk: no pipelining, and the budget taken from the first call
    _case(dev, rank, world, 300, 1, None, "single")
    os.environ.pop("FMSB_MOE_CHUNKS", None)
    print("DIST_OK moe_ep", flush=True)


def check_moe_library(dev, rank, world):
    """The same layer through library collectives (all_to_all_single on NCCL) and through the fused kernels."""
    from fms_acceleration_b200.ops import moe as MOE
    from fms_acceleration_b200.plugins.moe.utils.scattermoe import ScatterMoE

    H, I, E, k, T = 256, 128, 8 if 8 % world == 0 else 2 * world, 2, 384
    MOE.MoEContext._shared.clear()
    torch.manual_seed(3)
    mods = []
    for backend in ("fused", "library"):
        torch.manual_seed(3 + rank)
        m = ScatterMoE(H, "silu", I, E, top_k=k, dtype=torch.bfloat16, device=dev, ep_group=dist.group.WORLD)
        m.backend = backend
        with torch.no_grad():
            torch.manual_seed(5)
            m.router.weight.normal_(0, 0.05)
            torch.manual_seed(11 + rank)
            for w in (m.w1, m.w2, m.w3):
                w.weight.normal_(0, 0.05)
        mods.append(m)
    torch.manual_seed(50 + rank)
    x = (torch.randn(T, H, device=dev) * 0.5).bfloat16()
    outs = []
    for m in mods:
        xi = x.clone().requires_grad_()
        o, _ = m(xi)
        o.float().square().sum().backward()
        outs.append((o.detach().float(), xi.grad.float(), m.w2.weight.grad.float()))
    for a, b in zip(outs[0], outs[1]):
        assert ((a - b).norm() / b.norm().clamp(min=1e-9)).item() < 3e-2
    print("DIST_OK moe_library", flush=True)


def check_moe_lora(dev, rank, world):
    """Expert parallelism with per-expert LoRA: the fused path (low-rank pair inside the grouped GEMMs, two token
    slices) against the library path, which forms the dense W + A B; outputs, input and adapter gradients."""
    from types import SimpleNamespace

    from fms_acceleration_b200 import _native as NV
    from fms_acceleration_b200.ops import moe as MOE
    from fms_acceleration_b200.plugins.moe.utils.scattermoe import ScatterMoE

    H, I, E, k, T, r = 256, 128, 8 if 8 % world == 0 else 2 * world, 2, 384, 8
    os.environ["FMSB_MOE_CHUNKS"] = "2"
    MOE.MoEContext._shared.clear()
    mods = []
    for backend in ("fused", "library"):
        m = ScatterMoE(H, "silu", I, E, top_k=k, dtype=torch.bfloat16, device=dev, ep_group=dist.group.WORLD,
                       lora_config=SimpleNamespace(r=r, lora_alpha=r))
        m.backend = backend
        with torch.no_grad():
            torch.manual_seed(5)
            m.router.weight.normal_(0, 0.05)
            torch.manual_seed(11 + rank)
            for w in (m.w1, m.w2, m.w3):
                w.weight.normal_(0, 0.05)
                w.lora_A.normal_(0, 0.1)
                w.lora_B.normal_(0, 0.1)
        mods.append(m)
    torch.manual_seed(50 + rank)
    x = (torch.randn(T, H, device=dev) * 0.5).bfloat16()
    outs = []
    for m in mods:
        xi = x.clone().requires_grad_()
        o, _ = m(xi)
        o.float().square().sum().backward()
        assert m.w1.weight.grad is None
        outs.append([o.detach().float(), xi.grad.float()] +
                    [getattr(w, n).grad.float() for w in (m.w1, m.w2, m.w3) for n in ("lora_A", "lora_B")])
    NV.check_status()
    for i, (a, b) in enumerate(zip(outs[0], outs[1])):
        err = ((a - b).norm() / b.norm().clamp(min=1e-9)).item()
        assert err < 4e-2, (i, err)
    os.environ.pop("FMSB_MOE_CHUNKS", None)
    print("DIST_OK moe_lora", flush=True)
