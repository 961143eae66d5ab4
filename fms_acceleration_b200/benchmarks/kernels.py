"""Micro-benchmarks of the hand-written kernels with CUDA-event timing.

    python -m fms_acceleration_b200.benchmarks.kernels gemm --m 16384 --n 4096 --k 4096
    python -m fms_acceleration_b200.benchmarks.kernels attn --batch 4 --seq 4096
    python -m fms_acceleration_b200.benchmarks.kernels elementwise

Every number is taken after warm-up, with a synchronise on both sides, on inputs larger than the 126 MB L2 (or
with an L2 flush between iterations: ``--flush``).  ``--iters 1 --warmup 0`` gives a run suitable for profiling
one launch.  Results are printed as JSON lines; roofline fractions use ``MEASURED_PEAKS.json`` when present.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

REPO = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def peaks():
    p = os.path.join(REPO, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as fh:
            d = json.load(fh)
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


_flush_buf = None


def flush_l2():
    global _flush_buf
    if _flush_buf is None:
        _flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    _flush_buf.zero_()


def timeit(fn, iters, warmup, flush=False):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if not flush:
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(iters):
            fn()
        e.record()
        torch.cuda.synchronize()
        return s.elapsed_time(e) / iters
    total = 0.0
    for _ in range(iters):
        flush_l2()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        total += s.elapsed_time(e)
    return total / iters


def bench_gemm(a):
    from fms_acceleration_b200 import _native as NV
    from fms_acceleration_b200.ops.gemm import gemm

    pk = peaks()
    x = torch.randn(a.m, a.k, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(a.n, a.k, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(a.m, a.n, device="cuda", dtype=torch.bfloat16)
    b_mn = a.layout == "nn"
    wt = w.t().contiguous() if b_mn else w
    from fms_acceleration_b200.ops.gemm import set_pair_mode

    old = set_pair_mode(a.pair)
    t = timeit(lambda: gemm(x, wt, b_mn=b_mn, out=out), a.iters, a.warmup, a.flush)
    NV.check_status()
    fl = 2.0 * a.m * a.n * a.k
    res = {"kernel": "gemm_tcgen05", "m": a.m, "n": a.n, "k": a.k, "layout": a.layout, "pair_mode": a.pair, "ms": t,
           "tflops": fl / t / 1e9, "frac_of_%s_bf16_peak" % pk["source"]: fl / t / 1e9 / pk["bf16_tflops"]}
    import ctypes

    NV.declare("fmsb_gemm_pair_occupancy", [])
    res["pair_occupancy"] = int(NV.lib().fmsb_gemm_pair_occupancy())
    if a.both:
        set_pair_mode(0)
        t1 = timeit(lambda: gemm(x, wt, b_mn=b_mn, out=out), a.iters, a.warmup, a.flush)
        res["single_cta_ms"] = t1
        res["single_cta_tflops"] = fl / t1 / 1e9
    set_pair_mode(old)
    if a.cublas:
        t2 = timeit(lambda: torch.matmul(x, w.t(), out=out), a.iters, a.warmup, a.flush)
        res["cublas_ms"] = t2
        res["cublas_tflops"] = fl / t2 / 1e9
    print(json.dumps(res))


def bench_attn(a):
    from fms_acceleration_b200 import _native as NV
    from fms_acceleration_b200.ops import attention as AT
    from fms_acceleration_b200.trainer import synthetic_packed_batch

    nh, nkv, d = a.heads, a.kv_heads, a.head_dim
    T = a.batch * a.seq
    b = synthetic_packed_batch(32000, a.batch, a.seq, (128, a.seq), seed=1000, pin=False)
    cu = b["cu_seqlens"].cuda()
    ds, de = AT.doc_bounds_from_cu_seqlens(cu, T)
    lens = (cu[1:] - cu[:-1]).double()
    pairs = float((lens * (lens + 1) / 2).sum())
    fl_fwd = 4 * pairs * d * nh
    qkv = torch.randn(T, (nh + 2 * nkv) * d, device="cuda", dtype=torch.bfloat16)
    q, k, v = qkv[:, :nh * d], qkv[:, nh * d:(nh + nkv) * d], qkv[:, (nh + nkv) * d:]
    scale = d ** -0.5
    o, lse = AT._fwd(q, k, v, ds, de, nh, nkv, d, scale)
    do = torch.randn_like(o)
    t_f = timeit(lambda: AT._fwd(q, k, v, ds, de, nh, nkv, d, scale), a.iters, a.warmup, a.flush)
    t_b = timeit(lambda: AT._bwd(q, k, v, o, lse, do, ds, de, nh, nkv, d, scale), a.iters, a.warmup, a.flush)
    NV.check_status()
    extra = {}
    print(json.dumps({**extra, "kernel": "varlen_attention", "tokens": T, "heads": nh, "kv_heads": nkv, "head_dim": d,
                      "causal_pairs_per_head": pairs, "fwd_ms": t_f, "fwd_tflops": fl_fwd / t_f / 1e9, "bwd_ms": t_b,
                      "bwd_tflops": 2.5 * fl_fwd / t_b / 1e9}))


def bench_q4gemm(a):
    """Fused gather+dequant+GEMM+LoRA for few rows against dequantise-then-GEMM."""
    from fms_acceleration_b200 import _native as NV
    from fms_acceleration_b200.ops import quant as Q
    from fms_acceleration_b200.ops.gemm import gemm, gemm_q4_fused

    pk = peaks()
    Nn, K, R = a.n, a.k, 16
    w = (torch.randn(Nn, K, device="cuda") * 0.02).bfloat16()
    qs = Q.quantize_4bit(w, "nf4", 64, True)
    del w
    bl = (torch.randn(Nn, R, device="cuda") * 0.1).bfloat16()
    wd = torch.empty(Nn, K, dtype=torch.bfloat16, device="cuda")
    for M in a.rows:
        x = torch.randn(M, K, device="cuda").bfloat16()
        xa = torch.randn(M, R, device="cuda").bfloat16()

        def two_step():
            Q.dequantize_4bit(qs, torch.bfloat16, out=wd)
            return gemm(x, wd, a2=xa, b2=bl)

        t_f = timeit(lambda: gemm_q4_fused(x, qs, xa, bl), a.iters, a.warmup, True)
        t_2 = timeit(two_step, a.iters, a.warmup, True)
        NV.check_status()
        by = Nn * K / 2 + Nn * K / 64 + 2.0 * M * (K + Nn)
        print(json.dumps({"kernel": "gemm_q4_fused", "m": M, "n": Nn, "k": K, "lora_r": R, "fused_ms": t_f,
                          "dequant_then_gemm_ms": t_2, "speedup": t_2 / t_f, "algorithmic_gbs": by / t_f / 1e6,
                          "frac_of_%s_hbm" % pk["source"]: by / t_f / 1e6 / pk["hbm_gbs"],
                          "tflops": 2.0 * M * Nn * K / t_f / 1e9}))


def bench_elementwise(a):
    from fms_acceleration_b200.ops import activation as ACT
    from fms_acceleration_b200.ops import rmsnorm as RN

    pk = peaks()
    T, H, I = a.tokens, a.hidden, a.inter
    x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    w = torch.ones(H, device="cuda", dtype=torch.bfloat16)
    t = timeit(lambda: RN._fwd_native(x, w, 1e-6, False, None, False), a.iters, a.warmup, a.flush)
    by = 2.0 * T * H * 2
    print(json.dumps({"kernel": "rmsnorm_fwd", "ms": t, "gbs": by / t / 1e6, "frac_of_%s_hbm" % pk["source"]: by / t / 1e6 / pk["hbm_gbs"]}))
    y, _, inv = RN._fwd_native(x, w, 1e-6, False, None, False)
    t = timeit(lambda: RN._bwd_native(y, x, w, inv, False, None, False), a.iters, a.warmup, a.flush)
    by = 3.0 * T * H * 2
    print(json.dumps({"kernel": "rmsnorm_bwd", "ms": t, "gbs": by / t / 1e6, "frac_of_%s_hbm" % pk["source"]: by / t / 1e6 / pk["hbm_gbs"]}))
    gu = torch.randn(T, 2 * I, device="cuda", dtype=torch.bfloat16)
    t = timeit(lambda: ACT.glu_fwd(gu[:, :I], gu[:, I:], "silu"), a.iters, a.warmup, a.flush)
    by = 3.0 * T * I * 2
    print(json.dumps({"kernel": "swiglu_fwd", "ms": t, "gbs": by / t / 1e6, "frac_of_%s_hbm" % pk["source"]: by / t / 1e6 / pk["hbm_gbs"]}))


def _line(kernel, ms, nbytes, pk, **extra):
    d = {"kernel": kernel, "ms": ms, "gbs": nbytes / ms / 1e6,
         "frac_of_%s_hbm" % pk["source"]: nbytes / ms / 1e6 / pk["hbm_gbs"]}
    d.update(extra)
    print(json.dumps(d))


def bench_mamba(a):
    """Mamba2 pieces at the per-rank shape of the context-parallel benchmark (80 heads x 64, state 128, chunk 256):
    conv1d forward / backward, the decay-matrix builder, the masked head-sum of dG and the whole scan."""
    from fms_acceleration_b200 import _native as NV
    from fms_acceleration_b200.ops import mamba as MB

    pk = peaks()
    T, nh, P, G, N, Q = a.tokens, a.heads, a.head_dim, 1, a.state, a.chunk
    nc = T // Q
    dev, dt16 = "cuda", torch.bfloat16
    Cc = nh * P + 2 * G * N
    xc = torch.randn(T, Cc, device=dev, dtype=dt16)
    w = (torch.randn(Cc, 4, device=dev) * 0.5).to(dt16)
    b = torch.randn(Cc, device=dev, dtype=dt16)
    t = timeit(lambda: MB.causal_conv1d(xc, w, b), a.iters, a.warmup, a.flush)
    _line("conv1d_fwd", t, 2.0 * T * Cc * 2, pk)
    xg = xc.clone().requires_grad_()
    y = MB.causal_conv1d(xg, w, b)
    gy = torch.randn_like(y)
    t = timeit(lambda: torch.autograd.grad(y, xg, gy, retain_graph=True), a.iters, a.warmup, a.flush)
    _line("conv1d_bwd", t, 3.0 * T * Cc * 2, pk)
    # decay-matrix builder and masked head-sum on their own
    cb = torch.randn(nc * G * Q, Q, device=dev, dtype=dt16)
    dtv = torch.rand(T, nh, device=dev) * 0.05 + 0.001
    A = -(torch.rand(nh, device=dev) * 4 + 0.5)
    dtt = MB._chunk_major(dtv, nc, Q, nh)
    Lt = (dtt * A[None, :, None]).cumsum(-1)
    t = timeit(lambda: MB._make_g(cb, Lt, dtt, nc, nh, G, Q), a.iters, a.warmup, a.flush)
    _line("ssd_make_g2", t, nc * nh * Q * Q * 2.0, pk, note="bytes written; the lower triangle is computed, the rest zero-filled")
    dG = torch.randn(nc * nh * Q, Q, device=dev, dtype=dt16)
    dcb = torch.empty(nc * G * Q, Q, device=dev, dtype=dt16)

    def run_dcb():
        NV.check(NV.lib().fmsb_ssd_dcb(dG.data_ptr(), Lt.data_ptr(), dtt.data_ptr(), dcb.data_ptr(), nc, nh, G, Q,
                                       NV.dtype_code(dt16), NV.stream_ptr()), "fmsb_ssd_dcb")

    t = timeit(run_dcb, a.iters, a.warmup, a.flush)
    _line("ssd_dcb", t, nc * nh * Q * Q * 2.0 / 2, pk, note="bytes read: the lower triangle of dG")
    # whole scan
    x = (torch.randn(T, nh, P, device=dev) * 0.5).to(dt16).requires_grad_()
    B = (torch.randn(T, G, N, device=dev) * 0.3).to(dt16).requires_grad_()
    C = (torch.randn(T, G, N, device=dev) * 0.3).to(dt16).requires_grad_()
    D = torch.ones(nh, device=dev)
    dtp = dtv.clone().requires_grad_()
    t = timeit(lambda: MB.ssd_scan(x, dtp, A, B, C, D, None, Q), a.iters, a.warmup, a.flush)
    print(json.dumps({"kernel": "ssd_scan_fwd", "ms": t, "tokens": T}))
    yo, _ = MB.ssd_scan(x, dtp, A, B, C, D, None, Q)
    go = torch.randn_like(yo)
    t = timeit(lambda: torch.autograd.grad(yo, (x, dtp, B, C), go, retain_graph=True), a.iters, a.warmup, a.flush)
    print(json.dumps({"kernel": "ssd_scan_bwd", "ms": t, "tokens": T}))
    NV.check_status()


def bench_moe(a):
    """Single-GPU dispatch and combine of a Granite-3B-A800M layer (40 experts, top-8, hidden 1536)."""
    from fms_acceleration_b200 import _native as NV
    from fms_acceleration_b200.ops import moe as MOE

    pk = peaks()
    T, H, E, k = a.tokens, a.hidden, a.experts, a.top_k
    dev = torch.device("cuda", torch.cuda.current_device())
    x = torch.randn(T, H, device=dev, dtype=torch.bfloat16)
    g = torch.Generator(device=dev).manual_seed(0)
    idx = torch.rand(T, E, device=dev, generator=g).topk(k, dim=-1).indices.int().contiguous()
    wts = torch.full((T, k), 1.0 / k, device=dev)
    ctx = MOE.MoEContext(H, 512, E, k)
    cap = ctx.ensure(T, x.dtype, dev)
    seg_off, seg_cnt, dest_row = MOE._plan(ctx, idx, T, dev)
    t = timeit(lambda: MOE._plan(ctx, idx, T, dev), a.iters, a.warmup, a.flush)
    print(json.dumps({"kernel": "moe_plan (count + plan + 3-phase slot assignment)", "ms": t, "pairs": T * k}))
    buf, ptrs, _ = ctx._alloc("bench_recv", cap, H, x.dtype, dev)
    ld = buf.stride(0)
    t = timeit(lambda: MOE._dispatch(ctx, x, idx, dest_row, None, ptrs, ld), a.iters, a.warmup, a.flush)
    _line("moe_dispatch", t, (T * H + T * k * H) * 2.0, pk)
    t = timeit(lambda: MOE._combine(ctx, ptrs, ld, idx, dest_row, wts, T, H, x.dtype, dev), a.iters, a.warmup, a.flush)
    _line("moe_combine", t, (T * H + T * k * H) * 2.0, pk)
    NV.check_status()


def main(argv=None):
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="what", required=True)
    for name in ("gemm", "attn", "elementwise", "q4gemm", "mamba", "moe"):
        p = sub.add_parser(name)
        p.add_argument("--iters", type=int, default=20)
        p.add_argument("--warmup", type=int, default=5)
        p.add_argument("--flush", action="store_true", help="flush L2 between timed iterations")
        if name == "gemm":
            p.add_argument("--m", type=int, default=16384)
            p.add_argument("--n", type=int, default=4096)
            p.add_argument("--k", type=int, default=4096)
            p.add_argument("--layout", default="nt", choices=["nt", "nn"], help="nt: B is [N,K]; nn: B is [K,N]")
            p.add_argument("--cublas", action="store_true", help="also time torch.matmul (cuBLAS) for comparison")
            p.add_argument("--pair", type=int, default=1, help="CTA-pair kernel: 0 never, 1 by shape, 2 whenever possible")
            p.add_argument("--both", action="store_true", help="also time the single-CTA kernel")
        elif name == "q4gemm":
            p.add_argument("--n", type=int, default=14336)
            p.add_argument("--k", type=int, default=4096)
            p.add_argument("--rows", type=int, nargs="+", default=[16, 64, 128, 256, 512])
        elif name == "attn":
            p.add_argument("--batch", type=int, default=4)
            p.add_argument("--seq", type=int, default=4096)
            p.add_argument("--heads", type=int, default=32)
            p.add_argument("--kv-heads", type=int, default=8)
            p.add_argument("--head-dim", type=int, default=128)
        elif name == "mamba":
            p.add_argument("--tokens", type=int, default=8192)
            p.add_argument("--heads", type=int, default=80)
            p.add_argument("--head-dim", type=int, default=64)
            p.add_argument("--state", type=int, default=128)
            p.add_argument("--chunk", type=int, default=256)
        elif name == "moe":
            p.add_argument("--tokens", type=int, default=16384)
            p.add_argument("--hidden", type=int, default=1536)
            p.add_argument("--experts", type=int, default=40)
            p.add_argument("--top-k", type=int, default=8)
        else:
            p.add_argument("--tokens", type=int, default=16384)
            p.add_argument("--hidden", type=int, default=4096)
            p.add_argument("--inter", type=int, default=14336)
    a = ap.parse_args(argv)
    {"gemm": bench_gemm, "attn": bench_attn, "elementwise": bench_elementwise, "q4gemm": bench_q4gemm,
     "mamba": bench_mamba, "moe": bench_moe}[a.what](a)
    return 0


if __name__ == "__main__":
    sys.exit(main())
