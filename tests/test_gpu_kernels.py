"""Numerics of the hand-written sm_100a kernels against plain PyTorch fp32 references."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from fms_acceleration_b200 import _native as NV
from fms_acceleration_b200.ops import activation as A
from fms_acceleration_b200.ops import cross_entropy as CE
from fms_acceleration_b200.ops import quant as Q
from fms_acceleration_b200.ops import rmsnorm as RN
from fms_acceleration_b200.ops import rope as RP
from fms_acceleration_b200.ops.gemm import gemm

DEV = "cuda"


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp(min=1e-12)).item()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (200, 72, 136), (1000, 1032, 520)])
def test_gemm_layouts(dtype, a_mn, b_mn, M, N, K):
    torch.manual_seed(0)
    a = torch.randn((K, M) if a_mn else (M, K), device=DEV, dtype=dtype)
    b = torch.randn((K, N) if b_mn else (N, K), device=DEV, dtype=dtype)
    ref = (a.float().t() if a_mn else a.float()) @ (b.float() if b_mn else b.float().t())
    out = gemm(a, b, a_mn=a_mn, b_mn=b_mn)
    NV.check_status()
    assert out.shape == (M, N)
    assert _rel(out, ref) < 1e-2
    out32 = gemm(a, b, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32)
    NV.check_status()
    assert _rel(out32, ref) < 2e-3 if dtype == torch.float16 else _rel(out32, ref) < 2e-3


@pytest.mark.parametrize("bn", [16, 32, 64, 128, 256])
def test_gemm_tile_widths(bn):
    torch.manual_seed(1)
    M, N_, K = 384, 272, 320
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(N_, K, device=DEV, dtype=torch.bfloat16)
    out = gemm(a, b, bn=bn, out_dtype=torch.float32)
    NV.check_status()
    assert _rel(out, a.float() @ b.float().t()) < 2e-3


def test_gemm_dual_pair_and_epilogue():
    torch.manual_seed(2)
    M, N_, K, r = 512, 768, 1024, 16
    x = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(N_, K, device=DEV, dtype=torch.bfloat16) * 0.05
    xa = torch.randn(M, r, device=DEV, dtype=torch.bfloat16)
    lb = torch.randn(N_, r, device=DEV, dtype=torch.bfloat16)
    c = torch.randn(M, N_, device=DEV, dtype=torch.bfloat16)
    ref = 0.5 * (x.float() @ w.float().t() + xa.float() @ lb.float().t()) + 2.0 * c.float()
    out = gemm(x, w, a2=xa, b2=lb, c=c, alpha=0.5, beta=2.0, out_dtype=torch.float32)
    NV.check_status()
    assert _rel(out, ref) < 2e-3
    # in-place accumulate into a bf16 output
    d = c.clone()
    gemm(x, w, c=d, beta=1.0, out=d)
    NV.check_status()
    assert _rel(d, x.float() @ w.float().t() + c.float()) < 1e-2


def test_gemm_large_persistent():
    torch.manual_seed(3)
    M, N_, K = 4096, 4096, 2048
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(N_, K, device=DEV, dtype=torch.bfloat16)
    out = gemm(a, b)
    NV.check_status()
    ref = a @ b.t()
    assert _rel(out, ref) < 1e-2
    out2 = gemm(a, b)
    assert torch.equal(out, out2)


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("M,N_,K", [(512, 512, 256), (300, 520, 200), (1024, 768, 4096)])
def test_gemm_cta_pair_kernel(a_mn, b_mn, M, N_, K):
    """The CTA-pair kernel (256 x 256 tiles, tcgen05 cta_group::2) against the fp32 product and, bit for bit, against
    the single-CTA kernel (same contraction order); ragged M, N and K, all operand layouts, LoRA pair and C."""
    from fms_acceleration_b200.ops.gemm import set_pair_mode

    if (a_mn and M % 8) or (b_mn and N_ % 8):
        pytest.skip("MN-major operands need a leading dimension that is a multiple of 8")
    torch.manual_seed(4)
    a = torch.randn((K, M) if a_mn else (M, K), device=DEV, dtype=torch.bfloat16)
    b = torch.randn((K, N_) if b_mn else (N_, K), device=DEV, dtype=torch.bfloat16)
    ref = (a.float().t() if a_mn else a.float()) @ (b.float() if b_mn else b.float().t())
    old = set_pair_mode(0)
    try:
        single = gemm(a, b, a_mn=a_mn, b_mn=b_mn, bn=256, out_dtype=torch.float32)
        set_pair_mode(2)
        pair = gemm(a, b, a_mn=a_mn, b_mn=b_mn, bn=256, out_dtype=torch.float32)
        NV.check_status()
        assert _rel(pair, ref) < 2e-3
        assert torch.equal(pair, single)
        # 16-bit output: through shared memory and bulk tensor stores (ragged M / N are clipped by the store) and
        # through per-thread stores, bit for bit
        from fms_acceleration_b200.ops.gemm import set_pair_store

        staged = gemm(a, b, a_mn=a_mn, b_mn=b_mn, bn=256)
        old_store = set_pair_store(0)
        direct = gemm(a, b, a_mn=a_mn, b_mn=b_mn, bn=256)
        set_pair_store(old_store)
        NV.check_status()
        assert torch.equal(staged, direct)
        assert _rel(staged, ref) < 1e-2
        if not a_mn and not b_mn:
            r = 16
            xa = torch.randn(M, r, device=DEV, dtype=torch.bfloat16)
            lb = torch.randn(N_, r, device=DEV, dtype=torch.bfloat16)
            c = torch.randn(M, N_, device=DEV, dtype=torch.bfloat16)
            out = gemm(a, b, a2=xa, b2=lb, c=c, alpha=0.5, beta=2.0, bn=256)
            NV.check_status()
            want = 0.5 * (ref + xa.float() @ lb.float().t()) + 2.0 * c.float()
            assert _rel(out, want) < 1e-2
    finally:
        set_pair_mode(old)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rows,H", [(7, 256), (300, 4096), (33, 1536), (20011, 1024), (130, 2048), (5000, 2560), (10007, 4096),
                                    (3001, 5120), (1501, 8192), (9, 6144)])
def test_rmsnorm(dtype, rows, H):
    torch.manual_seed(0)
    x = torch.randn(rows, H, device=DEV, dtype=dtype, requires_grad=True)
    r = torch.randn(rows, H, device=DEV, dtype=dtype, requires_grad=True)
    w = (torch.randn(H, device=DEV, dtype=dtype) * 0.1 + 1).requires_grad_()
    y, h = RN.rmsnorm(x, w, 1e-6, False, r)
    gy = torch.randn_like(y)
    gh = torch.randn_like(h)
    (y.float() * gy.float()).sum().backward(retain_graph=True)
    # fp32 oracle
    xf, rf, wf = (t.detach().float().requires_grad_() for t in (x, r, w))
    hf = xf + rf
    yf = hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + 1e-6) * wf
    (yf * gy.float()).sum().backward()
    tol = 2e-2
    assert _rel(y, yf) < tol
    assert _rel(h, hf) < tol
    assert _rel(x.grad, xf.grad) < tol
    assert _rel(r.grad, rf.grad) < tol
    assert _rel(w.grad, wf.grad) < tol
    # no residual, gemma flavour
    x2 = torch.randn(rows, H, device=DEV, dtype=dtype)
    y2 = RN.rmsnorm(x2, w.detach(), 1e-5, True)
    ref2, _ = RN.rmsnorm_ref(x2.cpu(), w.detach().cpu(), 1e-5, True)
    assert _rel(y2.cpu(), ref2) < tol


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rows,H", [(37, 1024), (20011, 1024), (301, 1536), (130, 2048), (77, 2560), (300, 4096),
                                    (10007, 4096), (33, 5120), (2999, 8192), (45, 512), (11, 6144)])
@pytest.mark.parametrize("gemma", [False, True])
def test_rmsnorm_frozen_weight_paths(dtype, rows, H, gemma):
    """Frozen norm weight (adapter training): forward with and without the fused residual add and the backward that
    produces only the input / residual gradient, on every row width with a row-in-registers kernel, on widths that
    take the block-per-row kernels, and with more rows than one pass of the grid covers."""
    torch.manual_seed(rows + H)
    x = torch.randn(rows, H, device=DEV, dtype=dtype, requires_grad=True)
    r = torch.randn(rows, H, device=DEV, dtype=dtype, requires_grad=True)
    w = (torch.randn(H, device=DEV, dtype=dtype) * 0.1 + (0.0 if gemma else 1.0))
    y, h = RN.rmsnorm(x, w, 1e-6, gemma, r)
    gy, gh = torch.randn_like(y), torch.randn_like(h)
    torch.autograd.backward((y, h), (gy, gh))
    xf, rf = (t.detach().float().requires_grad_() for t in (x, r))
    hf = xf + rf
    hq = hf.detach().to(dtype).float() + (hf - hf.detach())  # the kernel normalises the stored (rounded) residual stream
    yf = hq * torch.rsqrt(hq.pow(2).mean(-1, keepdim=True) + 1e-6) * (w.float() + (1.0 if gemma else 0.0))
    torch.autograd.backward((yf, hf), (gy.float(), gh.float()))
    tol = 2e-2
    assert _rel(y, yf) < tol and _rel(h, hf) < tol
    assert _rel(x.grad, xf.grad) < tol and _rel(r.grad, rf.grad) < tol
    # no residual
    x2 = torch.randn(rows, H, device=DEV, dtype=dtype, requires_grad=True)
    y2 = RN.rmsnorm(x2, w, 1e-5, gemma)
    y2.backward(gy)
    x2f = x2.detach().float().requires_grad_()
    y2f = x2f * torch.rsqrt(x2f.pow(2).mean(-1, keepdim=True) + 1e-5) * (w.float() + (1.0 if gemma else 0.0))
    y2f.backward(gy.float())
    assert _rel(y2, y2f) < tol and _rel(x2.grad, x2f.grad) < tol


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_rope(dtype):
    torch.manual_seed(0)
    T, nh, d = 257, 6, 128
    x = torch.randn(T, nh, d, device=DEV, dtype=dtype, requires_grad=True)
    pos = torch.randint(0, 500, (T,), device=DEV, dtype=torch.int32)
    cos_t, sin_t = RP.rope_tables(d, 512, 10000.0, DEV)
    y = RP.apply_rope(x, pos, cos_t, sin_t)
    ref = RP.rope_ref(x.detach().float(), pos, cos_t, sin_t)
    assert _rel(y, ref) < 1e-2
    g = torch.randn_like(y)
    y.backward(g)
    gref = RP.rope_ref(g.float(), pos, cos_t, sin_t, -1.0)
    assert _rel(x.grad, gref) < 1e-2


@pytest.mark.parametrize("act", ["silu", "gelu", "gelu_pytorch_tanh"])
@pytest.mark.parametrize("rows,I", [(130, 1024), (3001, 24), (5, 14336), (70000, 520)])
def test_glu(act, rows, I):
    torch.manual_seed(0)
    eg = torch.randn(rows, 2 * I, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    e, g = eg[:, :I], eg[:, I:]
    h = A.glu(e, g, act)
    ef = eg.detach().float().requires_grad_()
    fn = {"silu": torch.nn.functional.silu, "gelu": torch.nn.functional.gelu,
          "gelu_pytorch_tanh": lambda t: torch.nn.functional.gelu(t, approximate="tanh")}[act]
    hf = fn(ef[:, :I]) * ef[:, I:]
    assert _rel(h, hf) < 1e-2
    gh = torch.randn_like(h)
    h.backward(gh)
    hf.backward(gh.float())
    assert _rel(eg.grad, ef.grad) < 1.5e-2


def test_glu_device_side_row_bound():
    """rows_dev: only the first n rows (a device scalar) are touched, forward and backward."""
    torch.manual_seed(1)
    rows, I, n = 300, 512, 123
    eg = torch.randn(rows, 2 * I, device=DEV, dtype=torch.bfloat16)
    used = torch.tensor([n], device=DEV, dtype=torch.int32)
    h = torch.full((rows, I), 7.0, device=DEV, dtype=torch.bfloat16)
    A.glu_fwd(eg[:, :I], eg[:, I:], "silu", out=h, rows_dev=used)
    ref = torch.nn.functional.silu(eg[:n, :I].float()) * eg[:n, I:].float()
    assert _rel(h[:n], ref) < 1e-2 and torch.all(h[n:] == 7.0)
    dh = torch.randn(rows, I, device=DEV, dtype=torch.bfloat16)
    de = torch.full((rows, I), 7.0, device=DEV, dtype=torch.bfloat16)
    dg = torch.full((rows, I), 7.0, device=DEV, dtype=torch.bfloat16)
    A.glu_bwd(dh, eg[:, :I], eg[:, I:], "silu", de=de, dg=dg, rows_dev=used)
    ef = eg[:n].float().requires_grad_()
    (torch.nn.functional.silu(ef[:, :I]) * ef[:, I:]).backward(dh[:n].float())
    assert _rel(de[:n], ef.grad[:, :I]) < 1.5e-2 and _rel(dg[:n], ef.grad[:, I:]) < 1.5e-2
    assert torch.all(de[n:] == 7.0) and torch.all(dg[n:] == 7.0)  # rows beyond the bound are not written


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("V", [1000, 32000, 70001])
def test_cross_entropy(dtype, V):
    torch.manual_seed(0)
    rows = 37
    logits = (torch.randn(rows, V, device=DEV) * 3).to(dtype).requires_grad_()
    labels = torch.randint(0, V, (rows,), device=DEV)
    labels[::5] = -100
    ref_in = logits.detach().float().requires_grad_()
    ref = torch.nn.functional.cross_entropy(ref_in, labels, ignore_index=-100, reduction="none")
    w = torch.randn(rows, device=DEV)
    (ref * w).sum().backward()
    keep = logits.detach().clone()
    loss = CE.fast_cross_entropy_loss(logits, labels)
    assert torch.allclose(loss, ref, rtol=1e-4, atol=1e-4)
    (loss * w).sum().backward()
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert _rel(logits.grad, ref_in.grad) < max(tol, 1e-5)
    # the backward reuses the logits storage for the gradient
    assert not torch.equal(keep, logits.detach()) or V == 0


def test_fused_linear_ce():
    torch.manual_seed(0)
    T, H, V = 700, 512, 4096
    x = (torch.randn(T, H, device=DEV) * 0.5).bfloat16().requires_grad_()
    w = (torch.randn(V, H, device=DEV) * 0.05).bfloat16().requires_grad_()
    labels = torch.randint(0, V, (T,), device=DEV)
    labels[:17] = -100
    loss = CE.fused_linear_cross_entropy(x, w, labels)
    NV.check_status()
    (loss * 2.0).backward()
    xf = x.detach().float().requires_grad_()
    wf = w.detach().float().requires_grad_()
    ref = torch.nn.functional.cross_entropy(xf @ wf.t(), labels, ignore_index=-100)
    (ref * 2.0).backward()
    assert abs(loss.item() - ref.item()) < 2e-2
    assert _rel(x.grad, xf.grad) < 3e-2
    assert _rel(w.grad, wf.grad) < 3e-2


@pytest.mark.parametrize("quant_type", ["nf4", "fp4"])
@pytest.mark.parametrize("double_quant", [True, False])
def test_quant4_roundtrip(quant_type, double_quant):
    torch.manual_seed(0)
    w = (torch.randn(512, 1024, device=DEV) * 0.02).bfloat16()
    qs = Q.quantize_4bit(w, quant_type, 64, double_quant)
    qs_ref = Q.quantize_4bit(w.cpu(), quant_type, 64, double_quant)
    # identical codes and scales as the CPU oracle
    assert (qs.packed.cpu() != qs_ref.packed).float().mean().item() < 1e-4
    if double_quant:
        assert (qs.absmax_q.cpu() != qs_ref.absmax_q).float().mean().item() < 1e-3
        assert torch.allclose(qs.absmax2.cpu(), qs_ref.absmax2)
    else:
        assert torch.allclose(qs.absmax.cpu(), qs_ref.absmax)
    for dt in (torch.bfloat16, torch.float16):
        d = Q.dequantize_4bit(qs, dt)
        d_ref = Q.dequantize_4bit_ref(qs.to("cpu"), dt)
        assert _rel(d.cpu(), d_ref) < 5e-3
    err = _rel(Q.dequantize_4bit(qs), w)
    assert err < (0.12 if quant_type == "nf4" else 0.2)


@pytest.mark.parametrize("bits", [2, 4, 8])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_gptq_dequant(bits, dtype):
    torch.manual_seed(0)
    i, o, gs = 512, 256, 128
    wi = torch.randint(0, 2 ** bits, (i, o), device=DEV)
    zi = torch.randint(0, 2 ** bits - 1, (i // gs, o), device=DEV)
    sc = (torch.rand(i // gs, o, device=DEV) * 0.01).to(dtype)
    qw, qz = Q.gptq_pack(wi, bits), Q.gptq_pack_zeros(zi, bits)
    g_idx = (torch.arange(i, device=DEV) // gs).int()
    for gi in (g_idx, None):
        for zoff in (0, 1):
            W = Q.gptq_dequant(qw, sc, qz, gi, bits, gs, zoff)
            ref = sc[g_idx.long()].float() * (wi - (zi[g_idx.long()] + zoff)).float()
            assert _rel(W, ref) < 5e-3
    # act-order style permuted groups
    perm = torch.randperm(i, device=DEV)
    g2 = g_idx[perm].contiguous()
    W = Q.gptq_dequant(qw, sc, qz, g2, bits, gs, 0)
    ref = sc[g2.long()].float() * (wi - zi[g2.long()]).float()
    assert _rel(W, ref) < 5e-3


@pytest.mark.parametrize("M,Nn,K,bn,double_quant,lora", [(64, 512, 256, 128, True, False), (128, 384, 512, 64, False, True),
                                                       (200, 256, 1024, 32, True, True), (7, 4096, 4096, None, True, True)])
def test_fused_q4_gemm_matches_dequant_then_gemm(M, Nn, K, bn, double_quant, lora):
    """In-kernel NF4 dequantisation (+ LoRA pair) against dequantise-to-bf16 followed by an fp32 matmul."""
    from fms_acceleration_b200.ops.gemm import gemm_q4_fused

    torch.manual_seed(M + Nn)
    w = torch.randn(Nn, K, device=DEV) * 0.05
    qs = Q.quantize_4bit(w.bfloat16(), "nf4", 64, double_quant)
    wd = Q.dequantize_4bit(qs, torch.bfloat16).view(Nn, K)
    x = (torch.randn(M, K, device=DEV) * 0.5).bfloat16()
    xa = bl = None
    ref = x.float() @ wd.float().t()
    if lora:
        xa = (torch.randn(M, 16, device=DEV) * 0.3).bfloat16()
        bl = (torch.randn(Nn, 16, device=DEV) * 0.3).bfloat16()
        ref = ref + xa.float() @ bl.float().t()
    y = gemm_q4_fused(x, qs, xa, bl, bn=bn)
    NV.check_status()
    assert y.shape == (M, Nn)
    assert (y.float() - ref).abs().max() <= 2e-2 * ref.abs().max() + 1e-3
    # several equal shards of the packed array addressed through a pointer table (here all on one GPU)
    import ctypes

    if (Nn * K // 2) % (4 * 32) == 0:
        sb = Nn * K // 2 // 4
        parts = [qs.packed[i * sb:(i + 1) * sb].clone() for i in range(4)]
        ptrs = (ctypes.c_void_p * 4)(*[t.data_ptr() for t in parts])
        y2 = gemm_q4_fused(x, qs, xa, bl, shard_ptrs=ptrs, shard_bytes=sb, bn=bn)
        NV.check_status()
        assert torch.equal(y2, y)


@pytest.mark.parametrize("M,Nn,K,gs,bn,dtype,zoff,lora", [(64, 512, 256, 128, 128, torch.float16, 0, False),
                                                         (128, 384, 512, 64, 64, torch.bfloat16, 1, True),
                                                         (200, 264, 1024, 1024, 32, torch.bfloat16, 0, True),
                                                         (5, 4096, 4096, 128, None, torch.float16, 1, False)])
def test_fused_gptq_gemm_matches_fp32_oracle(M, Nn, K, gs, bn, dtype, zoff, lora):
    """GPTQ int4 weights expanded inside the GEMM (+ LoRA pair) against the fp32 formula scale * (q - zero)."""
    from fms_acceleration_b200.ops.gemm import gemm_gptq_fused

    torch.manual_seed(M + Nn)
    wi = torch.randint(0, 16, (K, Nn), device=DEV)
    zi = torch.randint(0, 15, (K // gs, Nn), device=DEV)
    sc = (torch.rand(K // gs, Nn, device=DEV) * 0.02 + 0.001).to(dtype)
    qw, qz = Q.gptq_pack(wi, 4), Q.gptq_pack_zeros(zi, 4)
    g = (torch.arange(K, device=DEV) // gs).long()
    W = sc[g].float() * (wi - (zi[g] + zoff)).float()  # [K, N]
    x = (torch.randn(M, K, device=DEV) * 0.5).to(dtype)
    ref = x.float() @ W
    xa = bl = None
    if lora:
        xa = (torch.randn(M, 16, device=DEV) * 0.3).to(dtype)
        bl = (torch.randn(Nn, 16, device=DEV) * 0.3).to(dtype)
        ref = ref + xa.float() @ bl.float().t()
    y = gemm_gptq_fused(x, qw, sc, qz, gs, zoff, xa, bl, bn=bn)
    NV.check_status()
    assert y.shape == (M, Nn)
    assert (y.float() - ref).abs().max() <= 2e-2 * ref.abs().max() + 1e-3


def test_gptq_quantlinear_few_rows_uses_the_fused_kernel():
    """QuantLinear with a handful of rows: same numbers as dequantise-then-GEMM, forward and input gradient."""
    from fms_acceleration_b200.nn import gptq as G

    torch.manual_seed(4)
    q = G.QuantLinear.random(512, 384, bits=4, group_size=128, dtype=torch.float16, device=DEV, scale_std=0.01)
    x = (torch.randn(2, 5, 512, device=DEV) * 0.5).half().requires_grad_()
    assert q.fused_ok(x)
    y = q(x)
    y.float().square().sum().backward()
    NV.check_status()
    gx = x.grad.clone()
    x.grad = None
    saved = G.FUSED_Q4_MAX_ROWS
    G.FUSED_Q4_MAX_ROWS = 0
    try:
        assert not q.fused_ok(x)
        y2 = q(x)
        y2.float().square().sum().backward()
    finally:
        G.FUSED_Q4_MAX_ROWS = saved
    assert (y.float() - y2.float()).abs().max() <= 1e-2 * y2.float().abs().max() + 1e-3
    assert (gx.float() - x.grad.float()).abs().max() <= 2e-2 * x.grad.float().abs().max() + 1e-3


def test_linear4bit_few_rows_uses_the_fused_kernel():
    """Same numbers as the dequantise-then-GEMM path, forward and backward, for a handful of rows."""
    from fms_acceleration_b200.nn import Linear4bit
    from fms_acceleration_b200.nn import linear4bit as L4

    torch.manual_seed(3)
    lin = torch.nn.Linear(512, 384, bias=False, device=DEV, dtype=torch.bfloat16)
    q = Linear4bit.from_linear(lin, "nf4", 64, torch.bfloat16)
    x = (torch.randn(2, 5, 512, device=DEV) * 0.5).bfloat16().requires_grad_()
    y = q(x)
    y.float().square().sum().backward()
    NV.check_status()
    gx = x.grad.clone()
    x.grad = None
    saved = L4.FUSED_Q4_MAX_ROWS
    L4.FUSED_Q4_MAX_ROWS = 0
    try:
        y2 = q(x)
        y2.float().square().sum().backward()
    finally:
        L4.FUSED_Q4_MAX_ROWS = saved
    assert (y.float() - y2.float()).abs().max() <= 1e-2 * y2.float().abs().max() + 1e-3
    assert (gx.float() - x.grad.float()).abs().max() <= 2e-2 * x.grad.float().abs().max() + 1e-3


def test_fast_gemv_matches_dequantised_product():
    from fms_acceleration_b200.nn import Linear4bit
    from fms_acceleration_b200.ops.quant import fast_dequantize, fast_gemv

    torch.manual_seed(5)
    lin = torch.nn.Linear(1024, 768, bias=False, device=DEV, dtype=torch.bfloat16)
    q = Linear4bit.from_linear(lin, "nf4", 64, torch.bfloat16)
    x = (torch.randn(1, 3, 1024, device=DEV) * 0.5).bfloat16()
    y = fast_gemv(x, q)
    NV.check_status()
    w = fast_dequantize(q)
    ref = x.float() @ w.float().t()
    assert y.shape == (1, 3, 768)
    assert (y.float() - ref).abs().max() <= 1e-2 * ref.abs().max() + 1e-3


@pytest.mark.parametrize("M,Nn,K,dtype", [(48, 4096, 16384, torch.float32), (6144, 48, 8192, torch.float32),
                                          (1536, 512, 4096, torch.bfloat16)])
def test_weight_gradient_gemm_splits_the_contraction(M, Nn, K, dtype):
    """dW = dy^T x with few output tiles and a long token axis runs as slices of the contraction + one sum."""
    from fms_acceleration_b200.ops import gemm as GM

    torch.manual_seed(7)
    dy = (torch.randn(K, M, device=DEV) * 0.5).bfloat16()
    x = (torch.randn(K, Nn, device=DEV) * 0.5).bfloat16()
    assert GM._split_k(M, Nn, K, GM._pick_bn(Nn, True)) > 1
    out = GM.gemm(dy, x, a_mn=True, b_mn=True, out_dtype=dtype)
    NV.check_status()
    ref = dy.float().t() @ x.float()
    assert out.dtype == dtype and out.shape == (M, Nn)
    tol = 2e-3 if dtype == torch.float32 else 1e-2
    assert (out.float() - ref).abs().max() <= tol * ref.abs().max()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32, torch.float16])
@pytest.mark.parametrize("n", [8 * 1000 + 3, 1 << 20, 5])
def test_adamw_kernel_matches_torch_fused(dtype, n):
    """The in-tree AdamW step against torch's fused AdamW on the same parameters and gradients, three steps, with
    weight decay; sizes with a ragged tail and one smaller than a vector."""
    from fms_acceleration_b200.ops.optim import AdamW

    torch.manual_seed(n)
    w = torch.randn(n, device=DEV).to(dtype)
    a, b = w.clone().requires_grad_(), w.clone().requires_grad_()
    oa = AdamW([a], lr=3e-3, weight_decay=0.05)
    ob = torch.optim.AdamW([b], lr=3e-3, weight_decay=0.05, fused=True)
    for it in range(3):
        g = (torch.randn(n, device=DEV) * 0.1).to(dtype)
        a.grad, b.grad = g.clone(), g.clone()
        oa.step()
        ob.step()
    NV.check_status()
    tol = 1e-6 if dtype == torch.float32 else (8e-3 if dtype == torch.bfloat16 else 1e-3)
    assert (a.float() - b.float()).abs().max() <= tol * (1 + b.float().abs().max())
    sa, sb = oa.state[a], ob.state[b]
    assert _rel(sa["exp_avg"], sb["exp_avg"]) < 1e-2 and _rel(sa["exp_avg_sq"], sb["exp_avg_sq"]) < 1e-2
    # the clipping coefficient rides in the kernel
    oa.grad_scale = 0.5
    a2 = w.clone().requires_grad_()
    o2 = AdamW([a2], lr=3e-3, weight_decay=0.0)
    o2.grad_scale = 0.5
    b2 = w.clone().requires_grad_()
    o3 = torch.optim.AdamW([b2], lr=3e-3, weight_decay=0.0, fused=True)
    g = (torch.randn(n, device=DEV) * 0.1).to(dtype)
    a2.grad, b2.grad = g.clone(), (g.float() * 0.5).to(dtype)
    o2.step()
    o3.step()
    assert (a2.float() - b2.float()).abs().max() <= tol * (1 + b2.float().abs().max())
