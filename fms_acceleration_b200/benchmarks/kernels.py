"""Micro-benchmarks of the hand-written kernels with CUDA-event timing.

    python -m fms_acceleration_b200.benchmarks.kernels gemm --m 16384 --n 4096 --k 4096
    python -m fms_acceleration_b200.benchmarks.kernels attn --batch 4 --seq 4096
    python -m fms_acceleration_b200.benchmarks.kernels elementwise
    python -m fms_acceleration_b200.benchmarks.kernels grouped      # the grouped GEMMs of one MoE layer
    python -m fms_acceleration_b200.benchmarks.kernels reference    # beside the reference's Triton kernels / flash-attn

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
        from fms_acceleration_b200.ops.gemm import set_pair_store

        old_store = set_pair_store(0)
        t0 = timeit(lambda: gemm(x, wt, b_mn=b_mn, out=out), a.iters, a.warmup, a.flush)
        set_pair_store(old_store)
        res["pair_direct_store_ms"] = t0
        res["pair_direct_store_tflops"] = fl / t0 / 1e9
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
    dh = torch.randn(T, I, device="cuda", dtype=torch.bfloat16)
    de, dg = torch.empty_like(dh), torch.empty_like(dh)
    t = timeit(lambda: ACT.glu_bwd(dh, gu[:, :I], gu[:, I:], "silu", de=de, dg=dg), a.iters, a.warmup, a.flush)
    by = 5.0 * T * I * 2
    print(json.dumps({"kernel": "swiglu_bwd", "ms": t, "gbs": by / t / 1e6, "frac_of_%s_hbm" % pk["source"]: by / t / 1e6 / pk["hbm_gbs"]}))
    del gu, dh, de, dg
    # NF4 weight of the gate|up projection [2 * I, H] with double-quantised scales -> bf16 (0.5 + 2 bytes per value)
    from fms_acceleration_b200.ops import quant as Q

    wq = torch.randn(2 * I, H, device="cuda", dtype=torch.bfloat16) * 0.02
    qs = Q.quantize_4bit(wq, "nf4", 64, True)
    wd = torch.empty_like(wq)
    t = timeit(lambda: Q.dequantize_4bit(qs, torch.bfloat16, out=wd), a.iters, a.warmup, a.flush)
    by = 2.5 * wq.numel()
    print(json.dumps({"kernel": "dequant_nf4 [%d x %d]" % (2 * I, H), "ms": t, "gbs": by / t / 1e6,
                      "frac_of_%s_hbm" % pk["source"]: by / t / 1e6 / pk["hbm_gbs"]}))


def bench_grouped(a):
    """The grouped tcgen05 GEMMs of one Granite-3B-A800M expert layer (40 experts, top-8, hidden 1536, inter 512) on the
    expert-sorted layout: gate|up in one pass, down projection, the two weight-gradient products, the input gradient."""
    from fms_acceleration_b200 import _native as NV
    from fms_acceleration_b200.ops import moe as MOE

    T, H, I_, E, k = a.tokens, a.hidden, a.inter, a.experts, a.top_k
    dev = torch.device("cuda", torch.cuda.current_device())
    g = torch.Generator(device=dev).manual_seed(0)
    idx = torch.rand(T, E, device=dev, generator=g).topk(k, dim=-1).indices.int().contiguous()
    ctx = MOE.MoEContext(H, I_, E, k)
    cap = ctx.cap = (T * k + E * 128 + 127) // 128 * 128
    seg_off, seg_cnt, dest_row = MOE._plan(ctx, idx, T, dev)
    Xs = torch.randn(cap, H, device=dev, dtype=torch.bfloat16)
    w1, w3 = (torch.randn(E, H, I_, device=dev, dtype=torch.bfloat16) * 0.02 for _ in range(2))
    w2 = torch.randn(E, I_, H, device=dev, dtype=torch.bfloat16) * 0.02
    gu = torch.empty(cap, 2 * I_, device=dev, dtype=torch.bfloat16)
    hs = torch.randn(cap, I_, device=dev, dtype=torch.bfloat16)
    dY = torch.randn(cap, H, device=dev, dtype=torch.bfloat16)
    rows = T * k
    runs = [
        ("gate|up  [rows,H]x[H,2I] (one pass over A)", 2.0 * rows * H * 2 * I_,
         lambda: MOE.grouped_gemm(Xs, w1.view(E * H, I_), seg_off, E, mode=1, n=2 * I_, b_alt=w3.view(E * H, I_), out=gu)),
        ("down     [rows,I]x[I,H]", 2.0 * rows * I_ * H,
         lambda: MOE.grouped_gemm(hs, w2.view(E * I_, H), seg_off, E, mode=1, n=H)),
        ("dW gate|up  [H,rows]x[rows,2I] per expert", 2.0 * rows * H * 2 * I_,
         lambda: MOE.grouped_gemm(Xs, gu, seg_off, E, mode=2, m=H, n=2 * I_)),
        ("dW down  [I,rows]x[rows,H] per expert", 2.0 * rows * I_ * H,
         lambda: MOE.grouped_gemm(hs, dY, seg_off, E, mode=2, m=I_, n=H)),
        ("dX through gate and up (two operand pairs)", 2.0 * rows * 2 * I_ * H,
         lambda: MOE.grouped_gemm(gu[:, :I_], w1.view(E * H, I_), seg_off, E, mode=1, b_mn=False, n=H, a2=gu[:, I_:],
                                  b2=w3.view(E * H, I_))),
    ]
    for name, fl, fn in runs:
        t = timeit(fn, a.iters, a.warmup, a.flush)
        print(json.dumps({"kernel": "grouped_gemm " + name, "rows": rows, "ms": t, "tflops": fl / t / 1e9}))
    NV.check_status()


def bench_reference(a):
    """This package's kernels beside the reference's own Triton kernels (loaded by file path from the copy under
    baseline/_ref) and the installed flash-attn on the benchmark shapes: RMSNorm forward+backward, SwiGLU, fused
    linear + cross-entropy, varlen attention, one ScatterMoE expert layer."""
    from fms_acceleration_b200 import _native as NV
    from fms_acceleration_b200.baseline import backend as BK
    from fms_acceleration_b200.ops import activation as ACT
    from fms_acceleration_b200.ops import attention as AT
    from fms_acceleration_b200.ops import cross_entropy as CE
    from fms_acceleration_b200.ops import moe as MOE
    from fms_acceleration_b200.ops import rmsnorm as RN
    from fms_acceleration_b200.trainer import synthetic_packed_batch

    dev = torch.device("cuda", torch.cuda.current_device())
    T, H, I_, V = a.tokens, 4096, 14336, 32000
    Te = 4 * T  # rows of the element-wise comparisons: large enough that device time, not the host, is what is timed
    out = []

    def both(name, mine, ref):
        tm = timeit(mine, a.iters, a.warmup, a.flush)
        tr = timeit(ref, a.iters, a.warmup, a.flush) if ref is not None else None
        rec = {"op": name, "this_ms": tm, "reference_ms": tr, "speedup": (tr / tm) if tr else None}
        print(json.dumps(rec))
        out.append(rec)

    # RMSNorm forward + backward, hidden 4096
    rms = BK._load_reference("fms_acceleration_foak", "kernels.unsloth.rms_layernorm")
    norm = torch.nn.Module()
    # frozen, as the norms are under LoRA: the reference's kernel never forms a weight gradient
    norm.weight = torch.nn.Parameter(torch.ones(H, device=dev, dtype=torch.bfloat16), requires_grad=False)
    norm.variance_epsilon = 1e-6
    x = torch.randn(Te, H, device=dev, dtype=torch.bfloat16, requires_grad=True)
    gy = torch.randn(Te, H, device=dev, dtype=torch.bfloat16)

    def mine_rms():
        y = RN.rmsnorm(x, norm.weight, 1e-6)
        torch.autograd.grad(y, (x,), gy)

    def ref_rms():
        y = rms.fast_rms_layernorm(norm, x)
        torch.autograd.grad(y, (x,), gy)

    both(f"rmsnorm fwd+bwd [{Te}x{H}]", mine_rms, ref_rms)
    del x, gy
    # SwiGLU forward + backward, intermediate 14336
    glu = BK._load_reference("fms_acceleration_foak", "fused_ops.unsloth_lora.swiglu")
    e = torch.randn(Te, I_, device=dev, dtype=torch.bfloat16, requires_grad=True)
    g = torch.randn(Te, I_, device=dev, dtype=torch.bfloat16, requires_grad=True)
    gh = torch.randn(Te, I_, device=dev, dtype=torch.bfloat16)

    def mine_glu():
        h = ACT.glu(e, g, "silu")
        torch.autograd.grad(h, (e, g), gh)

    def ref_glu():
        h = BK._RefSwiGLU.apply(e, g, glu)
        torch.autograd.grad(h, (e, g), gh)

    both(f"swiglu fwd+bwd [{Te}x{I_}]", mine_glu, ref_glu)
    del e, g, gh
    # fused linear + cross entropy, vocabulary 32000
    lce = BK._load_reference("fms_acceleration_foak", "fused_ops.liger_ce.fused_linear_cross_entropy_loss")
    hid = torch.randn(T, H, device=dev, dtype=torch.bfloat16, requires_grad=True)
    wv = (torch.randn(V, H, device=dev, dtype=torch.bfloat16) * 0.02).requires_grad_()
    tgt = torch.randint(0, V, (T,), device=dev)

    def mine_lce():
        loss = CE.fused_linear_cross_entropy(hid, wv, tgt)
        torch.autograd.grad(loss, (hid,))

    def ref_lce():
        loss = lce.LigerFusedLinearCrossEntropyFunction.apply(hid, wv, tgt, None, -100, 0.0, "mean")
        torch.autograd.grad(loss, (hid,))

    both(f"fused linear+CE fwd+bwd [{T}x{H}] -> {V}", mine_lce, ref_lce)
    # varlen attention, 32 / 8 heads of 128
    from flash_attn import flash_attn_varlen_func

    nh, nkv, d = 32, 8, 128
    b = synthetic_packed_batch(V, 4, T // 4, (128, T // 4), seed=1000, pin=False)
    cu = b["cu_seqlens"].to(dev)
    ds, de = AT.doc_bounds_from_cu_seqlens(cu, T)
    q = torch.randn(T, nh, d, device=dev, dtype=torch.bfloat16, requires_grad=True)
    kk = torch.randn(T, nkv, d, device=dev, dtype=torch.bfloat16, requires_grad=True)
    vv = torch.randn(T, nkv, d, device=dev, dtype=torch.bfloat16, requires_grad=True)
    go = torch.randn(T, nh, d, device=dev, dtype=torch.bfloat16)
    mx = int((cu[1:] - cu[:-1]).max())

    def mine_attn():
        o = AT.varlen_attention(q, kk, vv, ds, de)
        torch.autograd.grad(o, (q, kk, vv), go)

    def ref_attn():
        o = flash_attn_varlen_func(q, kk, vv, cu, cu, mx, mx, causal=True)
        torch.autograd.grad(o, (q, kk, vv), go)

    both(f"varlen attention fwd+bwd [{T} tokens, {nh}/{nkv} heads x {d}]", mine_attn, ref_attn)
    # one Granite expert layer: 40 experts, top-8, hidden 1536, intermediate 512
    from fms_acceleration_b200.plugins.moe.utils.scattermoe import ScatterMoE

    ops = BK._load_reference("fms_acceleration_moe", "utils.scattermoe_utils.khd.kernels.ops")
    Hm, Im, E, k = 1536, 512, 40, 8
    moe = ScatterMoE(Hm, "silu", Im, E, top_k=k, dtype=torch.bfloat16, device=dev)
    with torch.no_grad():
        moe.router.weight.normal_(0, 0.02)
        for m in (moe.w1, moe.w2, moe.w3):
            m.weight.normal_(0, 0.02)
    xm = torch.randn(T, Hm, device=dev, dtype=torch.bfloat16, requires_grad=True)
    gm = torch.randn(T, Hm, device=dev, dtype=torch.bfloat16)
    runner = BK.BaselineRunner.__new__(BK.BaselineRunner)
    torch.nn.Module.__init__(runner)
    runner.k_moe = ops

    def mine_moe():
        o, _ = moe(xm)
        torch.autograd.grad(o, [xm] + list(moe.parameters()), gm)

    def ref_moe():
        o = runner._moe(moe, xm)
        torch.autograd.grad(o, [xm] + list(moe.parameters()), gm)

    both(f"ScatterMoE layer fwd+bwd [{T} tokens, {E} experts top-{k}, {Hm}/{Im}]", mine_moe, ref_moe)
    NV.check_status()
    del moe, xm, gm

    def guarded(name, build):
        """A comparison whose reference side has its own calling convention: a failure there is reported on the
        line instead of ending the run."""
        try:
            mine, ref = build()
            both(name, mine, ref)
        except Exception as exc:  # noqa: BLE001 - the reference's kernels are foreign code
            rec = {"op": name, "error": f"{type(exc).__name__}: {exc}"[:200]}
            print(json.dumps(rec))
            out.append(rec)

    # rotary embedding on q and k (32 + 8 heads x 128), forward + backward, one 4096-token sequence per batch row
    def build_rope():
        from fms_acceleration_b200.ops import rope as RP

        rope = BK._load_reference("fms_acceleration_foak", "kernels.unsloth.rope_embedding")
        B, S, nq, nk, hd = T // 4096, 4096, 32, 8, 128
        cos_t, sin_t = RP.rope_tables(hd, S, 10000.0, dev)
        pos = torch.arange(S, device=dev, dtype=torch.int32).repeat(B)
        q = torch.randn(B * S, nq, hd, device=dev, dtype=torch.bfloat16, requires_grad=True)
        kk = torch.randn(B * S, nk, hd, device=dev, dtype=torch.bfloat16, requires_grad=True)
        gq, gk = torch.randn_like(q), torch.randn_like(kk)
        # the reference takes [batch, heads, seq, dim] views and full-width cos / sin tables in the compute dtype
        cos_r = torch.cat([cos_t, cos_t], dim=-1).to(torch.bfloat16)
        sin_r = torch.cat([sin_t, sin_t], dim=-1).to(torch.bfloat16)
        q4 = q.detach().view(B, S, nq, hd).transpose(1, 2).requires_grad_()
        k4 = kk.detach().view(B, S, nk, hd).transpose(1, 2).requires_grad_()
        gq4, gk4 = gq.view(B, S, nq, hd).transpose(1, 2), gk.view(B, S, nk, hd).transpose(1, 2)

        def mine():
            a, b = RP.apply_rope(q, pos, cos_t, sin_t), RP.apply_rope(kk, pos, cos_t, sin_t)
            torch.autograd.grad((a, b), (q, kk), (gq, gk))

        def ref():
            a, b = rope.fast_rope_embedding(q4, k4, cos_r, sin_r)
            torch.autograd.grad((a, b), (q4, k4), (gq4, gk4))

        return mine, ref

    guarded(f"rope q,k fwd+bwd [{T} tokens, 32+8 heads x 128]", build_rope)

    # plain cross-entropy on materialised logits, vocabulary 32000
    def build_ce():
        ce = BK._load_reference("fms_acceleration_foak", "kernels.unsloth.cross_entropy_loss")
        logits = torch.randn(T, V, device=dev, dtype=torch.bfloat16, requires_grad=True)
        labels = torch.randint(0, V, (T,), device=dev)

        def mine():
            loss = CE.fast_cross_entropy_loss(logits, labels).sum() / T  # gradient over the logits, as the reference
            torch.autograd.grad(loss, logits)

        def ref():
            loss = ce.fast_cross_entropy_loss(logits.view(1, T, V), labels.view(1, T))
            torch.autograd.grad(loss, logits)

        return mine, ref

    guarded(f"cross-entropy fwd+bwd [{T} x {V}]", build_ce)

    # GPTQ int4 dequantisation of a 4096 x 14336 weight (group 128)
    def build_gptq():
        from fms_acceleration_b200.ops import quant as Q

        gk = BK._load_reference("fms_acceleration_foak", "fused_ops.unsloth_lora.gptq.triton.kernels")
        i_f, o_f, gs = 4096, 14336, 128
        wi = torch.randint(0, 16, (i_f, o_f), device=dev)
        zi = torch.randint(0, 15, (i_f // gs, o_f), device=dev)
        sc = (torch.rand(i_f // gs, o_f, device=dev) * 0.01).half()
        qw, qz = Q.gptq_pack(wi, 4), Q.gptq_pack_zeros(zi, 4)
        g_idx = (torch.arange(i_f, device=dev) // gs).int()
        outw = torch.empty(i_f, o_f, device=dev, dtype=torch.float16)

        def mine():
            Q.gptq_dequant(qw, sc, qz, None, 4, gs, 0, out=outw)

        def ref():
            gk.dequant248(qw, sc, qz, g_idx, 4)

        return mine, ref

    guarded("GPTQ int4 dequantise [4096 x 14336]", build_gptq)
    NV.check_status()
    return out


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
    cap = ctx.cap = (T * k + E * 128 + 127) // 128 * 128
    seg_off, seg_cnt, dest_row = MOE._plan(ctx, idx, T, dev)
    t = timeit(lambda: MOE._plan(ctx, idx, T, dev), a.iters, a.warmup, a.flush)
    print(json.dumps({"kernel": "moe_plan (count + plan + 3-phase slot assignment)", "ms": t, "pairs": T * k}))
    buf = torch.zeros(cap, H, dtype=x.dtype, device=dev)
    ptrs = MOE._one_ptr(buf)
    ld = buf.stride(0)
    t = timeit(lambda: MOE._dispatch(ctx, x, idx, dest_row, None, ptrs, ld), a.iters, a.warmup, a.flush)
    _line("moe_dispatch", t, (T * H + T * k * H) * 2.0, pk)
    t = timeit(lambda: MOE._combine(ctx, ptrs, ld, idx, dest_row, wts, T, H, x.dtype, dev), a.iters, a.warmup, a.flush)
    _line("moe_combine", t, (T * H + T * k * H) * 2.0, pk)
    NV.check_status()


def main(argv=None):
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="what", required=True)
    for name in ("gemm", "attn", "elementwise", "q4gemm", "mamba", "moe", "grouped", "reference"):
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
        elif name in ("moe", "grouped"):
            p.add_argument("--tokens", type=int, default=16384)
            p.add_argument("--hidden", type=int, default=1536)
            p.add_argument("--inter", type=int, default=512)
            p.add_argument("--experts", type=int, default=40)
            p.add_argument("--top-k", type=int, default=8)
        elif name == "reference":
            p.add_argument("--tokens", type=int, default=16384)
        else:
            p.add_argument("--tokens", type=int, default=16384)
            p.add_argument("--hidden", type=int, default=4096)
            p.add_argument("--inter", type=int, default=14336)
    a = ap.parse_args(argv)
    {"gemm": bench_gemm, "attn": bench_attn, "elementwise": bench_elementwise, "q4gemm": bench_q4gemm,
     "mamba": bench_mamba, "moe": bench_moe, "grouped": bench_grouped, "reference": bench_reference}[a.what](a)
    return 0


if __name__ == "__main__":
    sys.exit(main())
