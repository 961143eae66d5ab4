"""Mixture-of-experts kernels (router, plan, dispatch, grouped GEMM, combine) against a dense fp32 oracle."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from fms_acceleration_b200 import _native as NV
from fms_acceleration_b200.models.builder import build_model
from fms_acceleration_b200.ops import moe as MOE
from fms_acceleration_b200.plugins.moe.utils import prepare_scattermoe
from fms_acceleration_b200.plugins.moe.utils.scattermoe import ScatterMoE
from fms_acceleration_b200.trainer import synthetic_packed_batch, to_device

DEV = "cuda"


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp(min=1e-12)).item()


@pytest.mark.parametrize("E,k", [(8, 2), (40, 8), (96, 4)])
def test_router_topk(E, k):
    torch.manual_seed(0)
    T = 333
    logits = (torch.randn(T, E, device=DEV) * 2).requires_grad_()
    w, idx = MOE.router_topk(logits, k)
    p = torch.softmax(logits.detach().double(), -1)
    rw, ridx = torch.topk(p, k, dim=-1)
    rw = rw / rw.sum(-1, keepdim=True)
    assert torch.equal(idx.long().sort(-1).values, ridx.sort(-1).values)
    assert torch.allclose(w.double().sort(-1).values, rw.sort(-1).values, atol=1e-5)
    g = torch.randn(T, k, device=DEV)
    (w * g).sum().backward()
    lf = logits.detach().double().requires_grad_()
    pf = torch.softmax(lf, -1)
    sel = torch.gather(pf, 1, idx.long())
    sel = sel / sel.sum(-1, keepdim=True)
    (sel * g.double()).sum().backward()
    assert _rel(logits.grad, lf.grad) < 1e-4


@pytest.mark.parametrize("T,H,I,E,k", [(300, 256, 128, 8, 2), (1024, 1536, 512, 40, 8), (77, 512, 256, 16, 4)])
def test_scattermoe_matches_dense_oracle(T, H, I, E, k):
    torch.manual_seed(1)
    moe = ScatterMoE(H, "silu", I, E, top_k=k, dtype=torch.bfloat16, device=DEV)
    with torch.no_grad():
        moe.router.weight.normal_(0, 0.05)
        for m in (moe.w1, moe.w2, moe.w3):
            m.weight.normal_(0, 0.05)
    x = (torch.randn(T, H, device=DEV) * 0.5).bfloat16().requires_grad_()
    out, logits = moe(x)
    NV.check_status()
    _, kidx = MOE.router_topk(logits.detach(), k)
    g = torch.randn_like(out)
    out.backward(g)
    NV.check_status()
    # oracle (fp32, dense loop over experts) with the same routing decisions
    xf = x.detach().float().requires_grad_()
    ws = [p.detach().float().requires_grad_() for p in (moe.router.weight, moe.w1.weight, moe.w2.weight, moe.w3.weight)]
    ref, _ = MOE.moe_ref(xf, ws[0], ws[1], ws[2], ws[3], k, idx=kidx)
    ref.backward(g.float())
    assert _rel(out, ref) < 2e-2
    assert _rel(x.grad, xf.grad) < 3e-2
    for p, r, name in zip((moe.w1.weight, moe.w2.weight, moe.w3.weight), (ws[1], ws[2], ws[3]), "w1 w2 w3".split()):
        assert _rel(p.grad, r.grad) < 3e-2, name
    assert _rel(moe.router.weight.grad, ws[0].grad) < 6e-2


@pytest.mark.parametrize("T,H,I,E,k,r", [(300, 256, 128, 8, 2, 8), (1024, 1536, 512, 40, 8, 16), (77, 512, 256, 16, 4, 40)])
def test_expert_lora_rides_in_the_grouped_gemm(T, H, I, E, k, r):
    """Frozen expert weights with per-expert low-rank factors: the fused path (low-rank products as the second
    operand pair of the grouped GEMMs) against the fp32 dense ``W + A B`` oracle, outputs and all adapter gradients."""
    from types import SimpleNamespace

    torch.manual_seed(2)
    moe = ScatterMoE(H, "silu", I, E, top_k=k, dtype=torch.bfloat16, device=DEV,
                     lora_config=SimpleNamespace(r=r, lora_alpha=r))
    with torch.no_grad():
        moe.router.weight.normal_(0, 0.05)
        for m in (moe.w1, moe.w2, moe.w3):
            m.weight.normal_(0, 0.05)
            m.lora_A.normal_(0, 0.1)
            m.lora_B.normal_(0, 0.1)
    x = (torch.randn(T, H, device=DEV) * 0.5).bfloat16().requires_grad_()
    out, logits = moe(x)
    NV.check_status()
    _, kidx = MOE.router_topk(logits.detach(), k)
    g = torch.randn_like(out)
    out.backward(g)
    NV.check_status()
    assert moe.w1.weight.grad is None and moe.w2.weight.grad is None
    xf = x.detach().float().requires_grad_()
    rw = moe.router.weight.detach().float().requires_grad_()
    fac = {n: (getattr(moe, n).lora_A.detach().float().requires_grad_(), getattr(moe, n).lora_B.detach().float().requires_grad_())
           for n in ("w1", "w2", "w3")}
    dense = {n: getattr(moe, n).weight.detach().float() + torch.bmm(*fac[n]) for n in fac}
    ref, _ = MOE.moe_ref(xf, rw, dense["w1"], dense["w2"], dense["w3"], k, idx=kidx)
    ref.backward(g.float())
    assert _rel(out, ref) < 2e-2
    assert _rel(x.grad, xf.grad) < 3e-2
    for n in fac:
        assert _rel(getattr(moe, n).lora_A.grad, fac[n][0].grad) < 4e-2, n + ".lora_A"
        assert _rel(getattr(moe, n).lora_B.grad, fac[n][1].grad) < 4e-2, n + ".lora_B"
    assert _rel(moe.router.weight.grad, rw.grad) < 6e-2


@pytest.mark.parametrize("N,K,b_mn", [(1536, 512, True), (512, 1536, False), (1024, 1536, True), (264, 512, True)])
def test_grouped_gemm_store_epilogue_matches_plain_stores(N, K, b_mn):
    """Grouped-M GEMM: the epilogue through shared memory and bulk tensor stores gives the same bits as per-thread
    stores, with empty and single-tile segments, and both equal the fp32 product per segment."""
    from fms_acceleration_b200.ops.gemm import set_pair_store

    torch.manual_seed(N + K)
    E = 6
    tiles = [3, 0, 1, 5, 2, 0]
    off = [0]
    for t in tiles:
        off.append(off[-1] + 128 * t)
    rows = off[-1]
    seg_off = torch.tensor(off + [rows], dtype=torch.int32, device=DEV)
    a = (torch.randn(rows, K, device=DEV) * 0.5).bfloat16()
    w = (torch.randn(E, K, N, device=DEV) * 0.05).bfloat16() if b_mn else (torch.randn(E, N, K, device=DEV) * 0.05).bfloat16()
    outs = []
    for store in (1, 0):
        old = set_pair_store(store)
        try:
            out = torch.full((rows, N), 3.0, device=DEV, dtype=torch.bfloat16)
            MOE.grouped_gemm(a, w.view(-1, w.shape[2]), seg_off, E, mode=1, b_mn=b_mn, n=N, out=out)
            NV.check_status()
            outs.append(out)
        finally:
            set_pair_store(old)
    assert torch.equal(outs[0], outs[1])
    for e in range(E):
        r0, r1 = off[e], off[e + 1]
        if r1 > r0:
            ref = a[r0:r1].float() @ (w[e].float() if b_mn else w[e].float().t())
            assert _rel(outs[0][r0:r1], ref) < 1e-2


def test_granitemoe_fused_model_trains():
    torch.manual_seed(0)
    model = build_model("tiny-granitemoe", device=DEV, dtype=torch.bfloat16, seed=0)
    batch = synthetic_packed_batch(1024, 2, 256, (16, 256), seed=5, pin=False)
    ref = build_model("tiny-granitemoe", device="cpu", dtype=torch.float32, seed=0)
    ref.load_state_dict({k: v.float().cpu() for k, v in model.state_dict().items()})
    ref_loss = ref(**{k: v for k, v in batch.items() if k != "cu_seqlens"}).loss
    prepare_scattermoe(model, None, 0, 1, 1)
    model.enable_fused("fused_ce_liger")
    out = model(**{k: v for k, v in to_device(batch, DEV).items() if k != "cu_seqlens"})
    out.loss.backward()
    NV.check_status()
    assert abs(out.loss.item() - ref_loss.item()) < 5e-2
    grads = [p.grad for p in model.parameters() if p.requires_grad]
    assert all(g is not None and torch.isfinite(g).all() for g in grads)


def test_capacity_overflow_drops_rows_and_reports():
    """A receive buffer that is too small: excess (token, expert) pairs get slot -1, segment counts are clipped to
    the capacity, the overflow counter (not the status word, which later waits read as an abort signal) records
    it, and dispatch / combine touch nothing out of range."""
    torch.manual_seed(0)
    T, H, E, k = 512, 128, 4, 2
    ctx = MOE.MoEContext(H, 64, E, k)
    ctx.cap = 384  # instead of T*k + padding = 1024 + ...
    idx = torch.randint(0, E, (T, k), dtype=torch.int32, device=DEV)
    st = NV.status_word(DEV)
    st[0] = 0
    MOE.overflow_count(DEV, reset=True)
    seg_off, seg_cnt, dest_row = MOE._plan(ctx, idx, T, DEV)
    torch.cuda.synchronize()
    assert int(st[0].item()) == 0  # dropped rows do not make later bounded waits give up
    assert MOE.overflow_count(DEV, reset=True) > 0
    so, sc, dr = seg_off.cpu(), seg_cnt.cpu(), dest_row.cpu()
    assert int(so[-1]) <= ctx.cap and int(sc.sum()) <= ctx.cap
    kept = dr[dr >= 0]
    assert kept.numel() == int(sc.sum()) and kept.numel() < T * k
    assert kept.max() < ctx.cap and kept.unique().numel() == kept.numel()  # distinct, in-range slots
    for e in range(E):
        rows = dr[(idx.cpu() == e) & (dr >= 0)]
        assert rows.numel() == int(sc[e]) and (rows >= so[e]).all() and (rows < so[e] + sc[e]).all()
    # dispatch with a canary behind the buffer, then combine: dropped pairs contribute zero
    x = torch.randn(T, H, device=DEV).bfloat16()
    buf = torch.zeros(ctx.cap + 8, H, dtype=torch.bfloat16, device=DEV)
    buf[ctx.cap:] = 7.0
    import ctypes

    ptrs = (ctypes.c_void_p * 1)(buf.data_ptr())
    MOE._dispatch(ctx, x, idx, dest_row, None, ptrs, buf.stride(0))
    out = MOE._combine(ctx, ptrs, buf.stride(0), idx, dest_row, None, T, H, torch.bfloat16, DEV)
    torch.cuda.synchronize()
    assert (buf[ctx.cap:] == 7.0).all()
    n_kept = (dest_row >= 0).sum(1, keepdim=True).float()
    assert torch.allclose(out.float(), x.float() * n_kept, atol=0.08, rtol=0.02)
    NV.check_status()
