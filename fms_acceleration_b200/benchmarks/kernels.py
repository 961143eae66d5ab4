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
    t = timeit(lambda: gemm(x, wt, b_mn=b_mn, out=out), a.iters, a.warmup, a.flush)
    NV.check_status()
    fl = 2.0 * a.m * a.n * a.k
    res = {"kernel": "gemm_tcgen05", "m": a.m, "n": a.n, "k": a.k, "layout": a.layout, "ms": t,
           "tflops": fl / t / 1e9, "frac_of_%s_bf16_peak" % pk["source"]: fl / t / 1e9 / pk["bf16_tflops"]}
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
    if a.compare_v1:
        g3 = AT._bwd(q, k, v, o, lse, do, ds, de, nh, nkv, d, scale)
        for gen in (2,):
            AT.BWD_GENERATION = gen
            g = AT._bwd(q, k, v, o, lse, do, ds, de, nh, nkv, d, scale)
            extra[f"bwd_gen{gen}_ms"] = timeit(lambda: AT._bwd(q, k, v, o, lse, do, ds, de, nh, nkv, d, scale), a.iters,
                                               a.warmup, a.flush)
            extra[f"max_abs_diff_vs_gen{gen}"] = [float((x.float() - y.float()).abs().max()) for x, y in zip(g3, g)]
        AT.BWD_GENERATION = 3
        NV.check_status()
        extra["max_abs_grad"] = [float(y.float().abs().max()) for y in g3]
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


def main(argv=None):
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="what", required=True)
    for name in ("gemm", "attn", "elementwise", "q4gemm"):
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
            p.add_argument("--compare-v1", action="store_true", help="also run the earlier backward generations")
        else:
            p.add_argument("--tokens", type=int, default=16384)
            p.add_argument("--hidden", type=int, default=4096)
            p.add_argument("--inter", type=int, default=14336)
    a = ap.parse_args(argv)
    {"gemm": bench_gemm, "attn": bench_attn, "elementwise": bench_elementwise, "q4gemm": bench_q4gemm}[a.what](a)
    return 0


if __name__ == "__main__":
    sys.exit(main())
