"""Mamba2 kernels: conv1d and the chunked SSD scan (forward, backward, initial/final state) against the
sequential fp64 recurrence."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from fms_acceleration_b200 import _native as NV
from fms_acceleration_b200.ops import mamba as MB

DEV = "cuda"


def _rel(a, b):
    return ((a.double() - b.double()).norm() / b.double().norm().clamp(min=1e-12)).item()


def test_conv1d_matches_reference():
    torch.manual_seed(0)
    T, Cc = 300, 256
    x = torch.randn(T, Cc, device=DEV).bfloat16().requires_grad_()
    w = (torch.randn(Cc, 4, device=DEV) * 0.5).bfloat16().requires_grad_()
    b = torch.randn(Cc, device=DEV).bfloat16().requires_grad_()
    halo = torch.randn(3, Cc, device=DEV).bfloat16().requires_grad_()
    y = MB.causal_conv1d(x, w, b, halo)
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr, br, hr = (t.detach().float().requires_grad_() for t in (x, w, b, halo))
    yr = MB.conv1d_ref(xr, wr, br, hr)
    yr.backward(g.float())
    assert _rel(y, yr) < 1e-2
    assert _rel(x.grad, xr.grad) < 2e-2 and _rel(w.grad, wr.grad) < 2e-2
    assert _rel(b.grad, br.grad) < 2e-2 and _rel(halo.grad, hr.grad) < 2e-2
    # two dense outputs (channels [0, 64) and [64, C)): same numbers, same gradients
    x2, w2, b2, h2 = (t.detach().clone().requires_grad_() for t in (x, w, b, halo))
    ya, yb = MB.causal_conv1d(x2, w2, b2, h2, split=64)
    assert ya.shape == (T, 64) and yb.shape == (T, Cc - 64) and ya.is_contiguous() and yb.is_contiguous()
    assert torch.equal(torch.cat([ya, yb], 1), y)
    (ya.float() * g[:, :64].float()).sum().backward(retain_graph=True)
    (yb.float() * g[:, 64:].float()).sum().backward()
    NV.check_status()
    assert _rel(x2.grad, x.grad) < 1e-3 and _rel(w2.grad, w.grad) < 1e-3 and _rel(h2.grad, halo.grad) < 1e-3


def test_conv1d_packed_sequences_do_not_leak():
    """Three packed sequences: no tap reads across a boundary, forward and backward; fp16; no bias, no halo."""
    torch.manual_seed(1)
    T, Cc = 731, 264
    bounds = [0, 130, 131, 600, T]
    start = torch.empty(T, dtype=torch.int32)
    for a, b in zip(bounds[:-1], bounds[1:]):
        start[a:b] = a
    start = start.to(DEV)
    x = torch.randn(T, Cc, device=DEV).half().requires_grad_()
    w = (torch.randn(Cc, 4, device=DEV) * 0.5).half().requires_grad_()
    y = MB.causal_conv1d(x, w, None, None, start, None)
    g = torch.randn_like(y)
    y.backward(g)
    NV.check_status()
    xr, wr = (t.detach().float().requires_grad_() for t in (x, w))
    yr = MB.conv1d_ref(xr, wr, None, None, start)
    yr.backward(g.float())
    assert _rel(y, yr) < 1e-2
    assert _rel(x.grad, xr.grad) < 2e-2 and _rel(w.grad, wr.grad) < 2e-2


@pytest.mark.parametrize("T,nh,P,G,N,Q,with_h0", [(256, 4, 64, 1, 128, 64, False), (512, 8, 64, 2, 64, 128, True),
                                                  (512, 4, 64, 1, 128, 256, True)])
def test_ssd_scan_matches_recurrence(T, nh, P, G, N, Q, with_h0, monkeypatch):
    torch.manual_seed(0)
    if Q == 128:
        monkeypatch.setattr(MB, "SLAB_BYTES", nh * Q * Q * 4)  # one chunk per slab: the slab loop runs 4 times
    x = (torch.randn(T, nh, P, device=DEV) * 0.5).bfloat16().requires_grad_()
    dt = (torch.rand(T, nh, device=DEV) * 0.09 + 0.01).requires_grad_()
    A = (-(torch.rand(nh, device=DEV) * 3 + 0.5)).requires_grad_()
    B = (torch.randn(T, G, N, device=DEV) * 0.3).bfloat16().requires_grad_()
    C = (torch.randn(T, G, N, device=DEV) * 0.3).bfloat16().requires_grad_()
    D = torch.randn(nh, device=DEV).requires_grad_()
    h0 = (torch.randn(nh, P, N, device=DEV) * 0.2).requires_grad_() if with_h0 else None
    y, hT = MB.ssd_scan(x, dt, A, B, C, D, h0, Q, recompute=(Q == 256))  # one case rebuilds the states in the backward
    NV.check_status()
    gy, gh = torch.randn_like(y), torch.randn_like(hT) * 0.1
    ((y.float() * gy.float()).sum() + (hT * gh).sum()).backward()
    NV.check_status()
    ins = [t.detach().double().cpu().requires_grad_() for t in (x, dt, A, B, C, D)]
    h0r = h0.detach().double().cpu().requires_grad_() if with_h0 else None
    yr, hr = MB.ssd_ref(*ins, h0r)
    ((yr * gy.double().cpu()).sum() + (hr * gh.double().cpu()).sum()).backward()
    assert _rel(y.cpu(), yr) < 2e-2
    assert _rel(hT.cpu(), hr) < 2e-2
    names = ["x", "dt", "A", "B", "C", "D"]
    for n, t, r in zip(names, (x, dt, A, B, C, D), ins):
        assert _rel(t.grad.cpu(), r.grad) < 5e-2, (n, _rel(t.grad.cpu(), r.grad))
    if with_h0:
        assert _rel(h0.grad.cpu(), h0r.grad) < 5e-2


def test_mamba2_model_matches_cpu_reference():
    from fms_acceleration_b200.models.builder import build_model

    torch.manual_seed(0)
    model = build_model("tiny-mamba2", device=DEV, dtype=torch.bfloat16, seed=0)
    ref = build_model("tiny-mamba2", device="cpu", dtype=torch.float32, seed=0)
    ref.load_state_dict({k: v.float().cpu() for k, v in model.state_dict().items()})
    ids = torch.randint(0, 512, (1, 96))
    out = model(ids.to(DEV), labels=ids.to(DEV))
    out.loss.backward()
    NV.check_status()
    r = ref(ids, labels=ids)
    r.loss.backward()
    assert abs(out.loss.item() - r.loss.item()) < 3e-2
    rg = dict(ref.named_parameters())
    for n, p in model.named_parameters():
        if rg[n].grad is None or rg[n].grad.norm() < 1e-7:
            continue
        assert torch.isfinite(p.grad).all(), n
        if p.dim() < 2:
            # per-head scalars (dt_bias, A_log, D) and biases get gradients of order 1e-5 here, below what a bf16
            # forward resolves; their exact gradients are covered by test_ssd_scan_matches_recurrence
            continue
        assert _rel(p.grad.cpu(), rg[n].grad) < 0.1, (n, _rel(p.grad.cpu(), rg[n].grad))


def test_state_correction_matches_einsum():
    """Entering-state correction of context parallelism (tcgen05 products + fused element-wise kernels) against the
    einsum statement, forward and every gradient."""
    torch.manual_seed(2)
    T, nh, P, G, N, Q = 512, 8, 64, 2, 128, 128
    y0 = (torch.randn(T, nh, P, device=DEV) * 0.5).bfloat16().requires_grad_()
    h_in = (torch.randn(nh, P, N, device=DEV) * 0.3).requires_grad_()
    dt = (torch.rand(T, nh, device=DEV) * 0.02 + 0.001).requires_grad_()
    A = (-(torch.rand(nh, device=DEV) * 2 + 0.5)).requires_grad_()
    C = (torch.randn(T, G, N, device=DEV) * 0.3).bfloat16().requires_grad_()
    y = MB.state_correction(y0, h_in, dt, A, C, Q)
    NV.check_status()
    gy = torch.randn_like(y)
    (y.float() * gy.float()).sum().backward()
    NV.check_status()
    ins = [t.detach().double().requires_grad_() for t in (y0, h_in, dt, A, C)]
    yr = MB.state_correction_ref(*ins)
    (yr * gy.double()).sum().backward()
    assert _rel(y, yr) < 1e-2
    for n, t, r in zip(["y0", "h_in", "dt", "A", "C"], (y0, h_in, dt, A, C), ins):
        assert _rel(t.grad, r.grad) < 3e-2, (n, _rel(t.grad, r.grad))
