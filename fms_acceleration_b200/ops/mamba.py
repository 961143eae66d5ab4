"""Mamba2 operators: causal conv1d + SiLU and the chunked state-space-duality (SSD) scan, forward and backward.

GEMM-shaped work (C.B^T, G.X, chunk states, inter-chunk outputs and all their gradients) runs as uniform batched
tcgen05 GEMMs (``fmsb_batched_gemm``); the recurrence over chunks and the conv are CUDA kernels in
``csrc/mamba.cu``; every pass over a [chunks, heads, Q, Q] or [T, heads, P] tensor between the GEMMs is a kernel of
``csrc/mamba_scan.cu``; PyTorch only handles the [T, heads]-sized decay bookkeeping.  The scan takes an initial state and
returns the final state, which is the hook context parallelism uses (``parallel/context_parallel.py``).

Layouts: x [T, nh, P]; dt [T, nh] (after softplus, fp32); A [nh] (negative); B, C [T, G, N]; D [nh];
states [nh, P, N] fp32.  T must be a multiple of the chunk size Q.
"""
from __future__ import annotations

import ctypes

import torch
import torch.nn.functional as F

from .. import _native as NV
from .gemm import batched_gemm

P_, I_, L_, F_ = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
NV.declare("fmsb_conv1d_fwd", [P_, L_, P_, P_, P_, P_, P_, L_, P_, L_, I_, I_, I_, I_, I_, P_])
NV.declare("fmsb_conv1d_bwd", [P_, L_, P_, L_, I_, P_, L_, P_, P_, P_, P_, P_, L_, P_, P_, P_, I_, I_, I_, I_, P_])
NV.declare("fmsb_ssd_make_g2", [P_, P_, P_, P_, I_, I_, I_, I_, I_, P_])
NV.declare("fmsb_ssd_dcb", [P_, P_, P_, P_, I_, I_, I_, I_, I_, P_])
NV.declare("fmsb_ssd_rowscale", [P_, P_, P_, L_, I_, I_, P_])
NV.declare("fmsb_ssd_fwd_combine", [P_, P_, P_, P_, P_, P_, L_, I_, I_, I_, P_])
NV.declare("fmsb_ssd_addscaled", [P_, P_, P_, P_, L_, I_, I_, P_])
NV.declare("fmsb_ssd_rowdot", [P_, P_, P_, P_, L_, I_, I_, P_])
NV.declare("fmsb_ssd_bwd_combine", [P_, P_, P_, P_, P_, P_, P_, P_, P_, P_, P_, L_, I_, I_, I_, P_])
NV.declare("fmsb_ssd_state_fwd", [P_, P_, P_, P_, P_, I_, I_, I_, I_, P_])
NV.declare("fmsb_ssd_state_bwd", [P_, P_, P_, P_, P_, P_, P_, I_, I_, I_, I_, P_])


# ------------------------------------------------------------------------------------------------ oracles
def ssd_ref(x, dt, A, B, C, D, h0=None):
    """Sequential recurrence in fp64 (CPU oracle).  Returns (y [T,nh,P], final state [nh,P,N])."""
    T, nh, P = x.shape
    G, N = B.shape[1], B.shape[2]
    xd, dtd, Ad, Bd, Cd, Dd = (t.double() for t in (x, dt, A, B, C, D))
    rep = nh // G
    h = torch.zeros(nh, P, N, dtype=torch.float64, device=x.device) if h0 is None else h0.double().clone()
    ys = []
    for t in range(T):
        Bt = Bd[t].repeat_interleave(rep, 0)
        Ct = Cd[t].repeat_interleave(rep, 0)
        h = torch.exp(dtd[t] * Ad)[:, None, None] * h + dtd[t][:, None, None] * xd[t][:, :, None] * Bt[:, None, :]
        ys.append((h * Ct[:, None, :]).sum(-1) + Dd[:, None] * xd[t])
    return torch.stack(ys), h


def conv1d_ref(x, w, bias, halo=None, seq_start=None):
    """x [T, C]; w [C, K]; causal depthwise conv + SiLU (fp32 math)."""
    T, Cc = x.shape
    K = w.shape[1]
    xf = x.float()
    pad = torch.zeros(K - 1, Cc, dtype=torch.float32, device=x.device) if halo is None else halo.float()
    xp = torch.cat([pad, xf], 0)
    acc = bias.float()[None, :].expand(T, Cc).clone() if bias is not None else torch.zeros(T, Cc, device=x.device)
    for j in range(K):
        col = xp[j: j + T]
        if seq_start is not None:
            src = torch.arange(T, device=x.device) - (K - 1) + j
            col = torch.where((src >= seq_start.long())[:, None], col, torch.zeros_like(col))
        acc = acc + w.float()[:, j][None, :] * col
    return F.silu(acc).to(x.dtype)


# ------------------------------------------------------------------------------------------------ conv1d
def _vec_rows(t):
    """Rows with unit stride, a row step that is a multiple of 8 elements and a 16-byte aligned base."""
    if t.stride(1) == 1 and t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0:
        return t
    return t.contiguous()


class _CausalConv1d(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias, halo, seq_start, seq_end, split):
        T, Cc = x.shape
        K = w.shape[1]
        if Cc % 8 != 0 or K != 4 or split % 8 != 0:
            raise ValueError("the conv kernel needs 4 taps and channel counts that are multiples of 8")
        x = _vec_rows(x)
        two = 0 < split < Cc
        y = torch.empty(T, split if two else Cc, dtype=x.dtype, device=x.device)
        y2 = torch.empty(T, Cc - split, dtype=x.dtype, device=x.device) if two else None
        wc = w.contiguous()
        bc = None if bias is None else bias.contiguous()
        hc = None if halo is None else halo.contiguous()
        rc = NV.lib().fmsb_conv1d_fwd(x.data_ptr(), x.stride(0), wc.data_ptr(), NV.ptr(bc), NV.ptr(hc),
                                      NV.ptr(seq_start), y.data_ptr(), y.stride(0), NV.ptr(y2),
                                      y2.stride(0) if two else 0, split if two else Cc, T, Cc, K,
                                      NV.dtype_code(x.dtype), NV.stream_ptr())
        NV.check(rc, "fmsb_conv1d_fwd")
        ctx.save_for_backward(x, wc, bc, hc, seq_start)
        ctx.split = split if two else Cc
        if two:
            return y, y2
        return y, y.new_empty(0)

    @staticmethod
    def backward(ctx, dy, dy2):
        x, w, bias, halo, seq_start = ctx.saved_tensors
        T, Cc = x.shape
        K = w.shape[1]
        split = ctx.split
        two = split < Cc
        if dy is None:
            dy = torch.zeros(T, split, dtype=x.dtype, device=x.device)
        if two and dy2 is None:
            dy2 = torch.zeros(T, Cc - split, dtype=x.dtype, device=x.device)
        dy = _vec_rows(dy)
        dy2 = _vec_rows(dy2) if two else None
        dx = torch.empty(T, Cc, dtype=x.dtype, device=x.device)
        dhalo = torch.empty(K - 1, Cc, dtype=x.dtype, device=x.device) if halo is not None else None
        # tap and bias gradients are accumulated by the kernel: dw[c, j] = sum_t dpre[t, c] * xin[t - (K-1) + j, c]
        dwb = torch.zeros(Cc * (K + 1), dtype=torch.float32, device=x.device)
        dw32, db32 = dwb[: Cc * K].view(Cc, K), dwb[Cc * K:]
        rc = NV.lib().fmsb_conv1d_bwd(dy.data_ptr(), dy.stride(0), NV.ptr(dy2), dy2.stride(0) if two else 0, split,
                                      x.data_ptr(), x.stride(0), w.data_ptr(), NV.ptr(bias), NV.ptr(halo),
                                      NV.ptr(seq_start), dx.data_ptr(), dx.stride(0), NV.ptr(dhalo), dw32.data_ptr(),
                                      db32.data_ptr() if bias is not None else None, T, Cc, K, NV.dtype_code(x.dtype),
                                      NV.stream_ptr())
        NV.check(rc, "fmsb_conv1d_bwd")
        return dx, dw32.to(w.dtype), (db32.to(w.dtype) if bias is not None else None), dhalo, None, None, None


def causal_conv1d(x, w, bias=None, halo=None, seq_start=None, seq_end=None, split=None):
    """Depthwise causal conv (kernel 4) + SiLU on packed rows ``x [T, C]``; ``w [C, K]``.  With ``split`` the
    result comes back as two dense tensors, channels ``[0, split)`` and ``[split, C)`` (the scan wants its ``x``
    dense and ``B|C`` apart, so no copy is needed afterwards)."""
    if not x.is_cuda:
        y = conv1d_ref(x, w, bias, halo, seq_start)
        return y if split is None else (y[:, :split], y[:, split:])
    if split is None:
        return _CausalConv1d.apply(x, w, bias, halo, seq_start, seq_end, x.shape[1])[0]
    return _CausalConv1d.apply(x, w, bias, halo, seq_start, seq_end, split)


# ------------------------------------------------------------------------------------------------ SSD scan
def _rows16(t2):
    """The [T, heads*P] kernels use 16-byte accesses: make the base address fit (row lengths already do)."""
    return t2 if t2.data_ptr() % 16 == 0 and t2.is_contiguous() else t2.contiguous().clone()


def _chunk_major(v, nc, Q, nh):
    """[T, nh] fp32 -> [nc, nh, Q] contiguous (unit stride along the chunk for the Q x Q kernels)."""
    return v.view(nc, Q, nh).transpose(1, 2).contiguous()


def _make_g(cb, Lt, dtt, nc, nh, G, Q):
    g = torch.empty(nc * nh * Q, Q, dtype=cb.dtype, device=cb.device)
    rc = NV.lib().fmsb_ssd_make_g2(cb.data_ptr(), Lt.data_ptr(), dtt.data_ptr(), g.data_ptr(), nc, nh, G, Q,
                                   NV.dtype_code(cb.dtype), NV.stream_ptr())
    NV.check(rc, "fmsb_ssd_make_g2")
    return g


def _rowscale(x2, w, nh, P):
    """x2 [T, nh*P] (16-bit) times w [T, nh] (fp32), rounded back to 16 bits."""
    out = torch.empty_like(x2)
    rc = NV.lib().fmsb_ssd_rowscale(x2.data_ptr(), w.data_ptr(), out.data_ptr(), x2.shape[0] * nh, P,
                                    NV.dtype_code(x2.dtype), NV.stream_ptr())
    NV.check(rc, "fmsb_ssd_rowscale")
    return out


SLAB_BYTES = 1 << 30  # bound on the [chunks, heads, Q, Q] temporaries of the scan (counted at 4 bytes per value)


def _slabs(nc: int, nh: int, Q: int):
    """Ranges of chunks whose [chunks, heads, Q, Q] fp32 temporaries stay below ``SLAB_BYTES``."""
    step = max(1, SLAB_BYTES // (nh * Q * Q * 4))
    return [(c0, min(nc, c0 + step)) for c0 in range(0, nc, step)]


def _chunk_states(x2, dt, A, B2, C2, h0, T, nh, P, G, N, Q, dtp, dev, cp=None, want_zero_start=False):
    """Decay bookkeeping and the state entering every chunk: (L, Ltot, cb, wgt, hprev, hT).  Shared by the forward
    and, with ``recompute``, by the backward (which then keeps none of these between the two passes).

    ``cp`` (context parallelism): once the chunk states are known, ``cp.forward`` runs the zero-start recurrence whose
    kernel hands this slice's final state to the later ranks, and returns the state ENTERING this slice; the
    recurrence proper then starts from it.  Two more values are returned in that case: the entering state and the
    zero-start entering states of the chunks (``want_zero_start`` asks for the latter without any exchange)."""
    nc, hpg = T // Q, nh // G
    # within-chunk cumulative sum of dt*A, taken along the unit-stride axis of the chunk-major layout
    dtt = _chunk_major(dt, nc, Q, nh)
    Lt = (dtt * A.float()[None, :, None]).cumsum(-1)                        # [nc, nh, Q]
    L = Lt.transpose(1, 2).reshape(T, nh).contiguous()
    Ltot = Lt[:, :, -1].contiguous()                                        # [nc, nh]
    # C.B^T per chunk and group
    cb = batched_gemm(C2, B2, M=Q, N=Q, K=N, n_batch=nc * G, n_inner=G, a_off=(Q, 0, N, 1), b_off=(Q, 0, N, 1),
                      d_off=(G * Q, Q, 0), out_rows=nc * G * Q, out_cols=Q)
    # chunk states S[c,h] [P, N] = (x w)^T B,  w = exp(Ltot - L) dt
    wgt = (torch.exp(Ltot.view(nc, 1, nh) - L.view(nc, Q, nh)) * dt.view(nc, Q, nh)).reshape(T, nh).contiguous()
    xw = _rowscale(x2, wgt, nh, P)
    S = batched_gemm(xw, B2, M=P, N=N, K=Q, n_batch=nc * nh, n_inner=nh, a_off=(Q, 0, P, 1), b_off=(Q, 0, N, hpg),
                     d_off=(nh * P, P, 0), a_mn=True, b_mn=True, out_rows=nc * nh * P, out_cols=N,
                     out_dtype=torch.float32)
    del xw
    hprev0 = None
    if cp is not None:
        hprev0 = torch.empty(nc * nh * P, N, dtype=dtp, device=dev)
        h0 = cp.forward(S, Ltot, hprev0, nc, nh, P * N, dtp)
    elif want_zero_start:
        hprev0 = torch.empty(nc * nh * P, N, dtype=dtp, device=dev)
        scratch = torch.empty(nh, P, N, dtype=torch.float32, device=dev)
        rc = NV.lib().fmsb_ssd_state_fwd(S.data_ptr(), Ltot.data_ptr(), None, hprev0.data_ptr(), scratch.data_ptr(), nc,
                                         nh, P * N, NV.dtype_code(dtp), NV.stream_ptr())
        NV.check(rc, "fmsb_ssd_state_fwd")
    hprev = torch.empty(nc * nh * P, N, dtype=dtp, device=dev)
    hT = torch.empty(nh, P, N, dtype=torch.float32, device=dev)
    h0c = None if h0 is None else h0.float().contiguous()
    rc = NV.lib().fmsb_ssd_state_fwd(S.data_ptr(), Ltot.data_ptr(), NV.ptr(h0c), hprev.data_ptr(), hT.data_ptr(), nc,
                                     nh, P * N, NV.dtype_code(dtp), NV.stream_ptr())
    NV.check(rc, "fmsb_ssd_state_fwd")
    if cp is not None or want_zero_start:
        return L, Ltot, Lt, dtt, cb, wgt, hprev, hT, h0c, hprev0
    return L, Ltot, Lt, dtt, cb, wgt, hprev, hT


class _SSDScan(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dt, A, B, C, D, h0, Q, recompute, cp=None):
        T, nh, P = x.shape
        G, N = B.shape[1], B.shape[2]
        assert T % Q == 0, "sequence length must be a multiple of the chunk size"
        assert Q % 8 == 0 and 256 % (Q // 8) == 0 and Q <= 1024 and P % 8 == 0, \
            "chunk size must be 8 times a divisor of 256, at most 1024 (32 ... 256, 512, 1024) and the head dimension a multiple of 8"
        nc, hpg = T // Q, nh // G
        dev, dtp = x.device, x.dtype
        x2 = _rows16(x.reshape(T, nh * P))
        B2, C2 = B.reshape(T, G * N), C.reshape(T, G * N)
        dt = dt.float().contiguous()
        h_in = hprev0 = None
        if cp is not None:
            assert h0 is None, "the entering state of a context-parallel slice comes from the earlier ranks"
            L, Ltot, Lt, dtt, cb, wgt, hprev, hT, h_in, hprev0 = _chunk_states(x2, dt, A, B2, C2, None, T, nh, P, G, N,
                                                                              Q, dtp, dev, cp=cp)
        else:
            L, Ltot, Lt, dtt, cb, wgt, hprev, hT = _chunk_states(x2, dt, A, B2, C2, h0, T, nh, P, G, N, Q, dtp, dev)
        # intra-chunk term in slabs of chunks: the [chunks, heads, Q, Q] decay-weighted matrices are transient
        y_intra = torch.empty(T, nh * P, dtype=torch.float32, device=dev)
        for c0, c1 in _slabs(nc, nh, Q):
            n = c1 - c0
            g = _make_g(cb[c0 * G * Q: c1 * G * Q], Lt[c0:c1], dtt[c0:c1], n, nh, G, Q)     # [n*nh*Q, Q]
            batched_gemm(g, x2[c0 * Q: c1 * Q], M=Q, N=P, K=Q, n_batch=n * nh, n_inner=nh, a_off=(nh * Q, Q, 0, 1),
                         b_off=(Q, 0, P, 1), d_off=(Q, 0, P), b_mn=True, out=y_intra[c0 * Q: c1 * Q])
            del g
        # inter-chunk: C_t . Hprev[c,h]  (B operand [P rows, N cols], contraction over N)
        y_inter = batched_gemm(C2, hprev, M=Q, N=P, K=N, n_batch=nc * nh, n_inner=nh, a_off=(Q, 0, N, hpg),
                               b_off=(nh * P, P, 0, 1), d_off=(Q, 0, P), out_rows=T, out_cols=nh * P,
                               out_dtype=torch.float32)
        # y = y_intra + exp(L) y_inter + D x
        y = torch.empty(T, nh, P, dtype=dtp, device=dev)
        Df = D.float().contiguous()
        rc = NV.lib().fmsb_ssd_fwd_combine(y_intra.data_ptr(), y_inter.data_ptr(), x2.data_ptr(), L.data_ptr(),
                                           Df.data_ptr(), y.data_ptr(), T * nh, P, nh, NV.dtype_code(dtp),
                                           NV.stream_ptr())
        NV.check(rc, "fmsb_ssd_fwd_combine")
        if recompute:
            # keep the inputs only; the backward rebuilds the bookkeeping and the entering states (under context
            # parallelism from the entering state received in the forward: nothing is exchanged a second time)
            ctx.save_for_backward(x, dt, A, B, C, D, h_in if cp is not None else h0)
        elif cp is not None:
            ctx.save_for_backward(x, dt, A, B, C, D, L, Ltot, cb, hprev, wgt, hprev0)
        else:
            ctx.save_for_backward(x, dt, A, B, C, D, L, Ltot, cb, hprev, wgt)
        ctx.meta = (Q, h0 is not None, recompute)
        ctx.cp = cp
        return y, hT

    @staticmethod
    def backward(ctx, dy, dhT):
        Q, has_h0, recompute = ctx.meta
        saved = ctx.saved_tensors  # read once: activation checkpointing allows a single unpack
        x, dt, A, B, C, D = saved[:6]
        T, nh, P = x.shape
        G, N = B.shape[1], B.shape[2]
        nc, hpg = T // Q, nh // G
        dev, dtp = x.device, x.dtype
        code = NV.dtype_code(dtp)
        x2 = _rows16(x.reshape(T, nh * P))
        B2, C2 = B.reshape(T, G * N), C.reshape(T, G * N)
        dy2 = _rows16(dy.reshape(T, nh * P))
        cp = ctx.cp
        hprev0 = None
        if recompute and cp is not None:
            L, Ltot, Lt, dtt, cb, wgt, hprev, _, _, hprev0 = _chunk_states(x2, dt, A, B2, C2, saved[6], T, nh,
                                                                         P, G, N, Q, dtp, dev, want_zero_start=True)
        elif recompute:
            L, Ltot, Lt, dtt, cb, wgt, hprev, _ = _chunk_states(x2, dt, A, B2, C2, saved[6], T, nh, P, G, N,
                                                                Q, dtp, dev)
        else:
            if cp is not None:
                L, Ltot, cb, hprev, wgt, hprev0 = saved[6:]
            else:
                L, Ltot, cb, hprev, wgt = saved[6:]
            Lt, dtt = _chunk_major(L, nc, Q, nh), _chunk_major(dt, nc, Q, nh)
        # ---- inter-chunk term  y += exp(L) * (C . Hprev)
        dyi = _rowscale(dy2, torch.exp(L), nh, P)
        y_inter = batched_gemm(C2, hprev, M=Q, N=P, K=N, n_batch=nc * nh, n_inner=nh, a_off=(Q, 0, N, hpg),
                               b_off=(nh * P, P, 0, 1), d_off=(Q, 0, P), out_rows=T, out_cols=nh * P,
                               out_dtype=torch.float32)
        # dC_inter[c, g] [Q, N] = dyi[c, heads of g] [Q, hpg*P] . Hprev[c, heads of g] [(h,p), N]
        dC = batched_gemm(dyi, hprev, M=Q, N=N, K=hpg * P, n_batch=nc * G, n_inner=G, a_off=(Q, 0, hpg * P, 1),
                          b_off=(nh * P, hpg * P, 0, 1), d_off=(Q, 0, N), b_mn=True, out_rows=T, out_cols=G * N,
                          out_dtype=torch.float32)
        # dHprev_direct[c,h] [P, N] = dyi[c,h]^T C[c]
        dhp = batched_gemm(dyi, C2, M=P, N=N, K=Q, n_batch=nc * nh, n_inner=nh, a_off=(Q, 0, P, 1), b_off=(Q, 0, N, hpg),
                           d_off=(nh * P, P, 0), a_mn=True, b_mn=True, out_rows=nc * nh * P, out_cols=N,
                           out_dtype=torch.float32)
        del dyi
        # ---- recurrence backward
        dS16 = torch.empty(nc * nh * P, N, dtype=dtp, device=dev)
        dh0 = torch.empty(nh, P, N, dtype=torch.float32, device=dev) if (has_h0 or cp is not None) else None
        dLtot = torch.zeros(nc, nh, dtype=torch.float32, device=dev)
        dhTc = None if dhT is None else dhT.float().contiguous()
        rc = NV.lib().fmsb_ssd_state_bwd(dhp.data_ptr(), NV.ptr(dhTc), Ltot.data_ptr(), hprev.data_ptr(),
                                         dS16.data_ptr(), NV.ptr(dh0), dLtot.data_ptr(), nc, nh, P * N, code,
                                         NV.stream_ptr())
        NV.check(rc, "fmsb_ssd_state_bwd")
        del dhp
        if cp is not None:
            # dh0 is the gradient of the state that ENTERED this slice: it belongs to the final states and decays of
            # the earlier ranks.  In return the later ranks send the gradient of THIS slice's zero-start final state
            # and total log-decay; it runs back through the zero-start recurrence (same decays, zero-start states).
            dF, dlogP = cp.backward(dh0, nh, P * N)
            dS16b = torch.empty_like(dS16)
            rc = NV.lib().fmsb_ssd_state_bwd(None, dF.data_ptr(), Ltot.data_ptr(), hprev0.data_ptr(), dS16b.data_ptr(),
                                             None, dLtot.data_ptr(), nc, nh, P * N, code, NV.stream_ptr())
            NV.check(rc, "fmsb_ssd_state_bwd")
            dS16 += dS16b
            del dS16b
            dLtot += dlogP[None, :]
            dh0 = None
        # ---- chunk state  S = (x w)^T B
        xw = _rowscale(x2, wgt, nh, P)
        # dXw[c,h] [Q, P] = B[c] [Q, N] . dS[c,h]^T
        dxw = batched_gemm(B2, dS16, M=Q, N=P, K=N, n_batch=nc * nh, n_inner=nh, a_off=(Q, 0, N, hpg),
                           b_off=(nh * P, P, 0, 1), d_off=(Q, 0, P), out_rows=T, out_cols=nh * P,
                           out_dtype=torch.float32)
        # dB_state[c, g] [Q, N] = xw[c, heads of g] [Q, hpg*P] . dS[c, heads of g] [(h,p), N]
        dB = batched_gemm(xw, dS16, M=Q, N=N, K=hpg * P, n_batch=nc * G, n_inner=G, a_off=(Q, 0, hpg * P, 1),
                          b_off=(nh * P, hpg * P, 0, 1), d_off=(Q, 0, N), b_mn=True, out_rows=T, out_cols=G * N,
                          out_dtype=torch.float32)
        del xw, dS16
        # ---- intra-chunk term  y += G X,  G = CB o exp(L_t - L_s) dt_s (s <= t); slabs of chunks bound the
        # [chunks, heads, Q, Q] temporaries
        dx_intra = torch.empty(T, nh * P, dtype=torch.float32, device=dev)
        y_intra = torch.empty(T, nh * P, dtype=torch.float32, device=dev)
        for c0, c1 in _slabs(nc, nh, Q):
            n = c1 - c0
            rows = slice(c0 * Q, c1 * Q)
            g = _make_g(cb[c0 * G * Q: c1 * G * Q], Lt[c0:c1], dtt[c0:c1], n, nh, G, Q)
            batched_gemm(g, dy2[rows], M=Q, N=P, K=Q, n_batch=n * nh, n_inner=nh, a_off=(nh * Q, Q, 0, 1),
                         b_off=(Q, 0, P, 1), d_off=(Q, 0, P), a_mn=True, b_mn=True, out=dx_intra[rows])
            batched_gemm(g, x2[rows], M=Q, N=P, K=Q, n_batch=n * nh, n_inner=nh, a_off=(nh * Q, Q, 0, 1),
                         b_off=(Q, 0, P, 1), d_off=(Q, 0, P), b_mn=True, out=y_intra[rows])
            del g
            dG = batched_gemm(dy2[rows], x2[rows], M=Q, N=Q, K=P, n_batch=n * nh, n_inner=nh, a_off=(Q, 0, P, 1),
                              b_off=(Q, 0, P, 1), d_off=(nh * Q, Q, 0), out_rows=n * nh * Q, out_cols=Q)
            # dCB[c, g] = sum_{h in g} dG o exp(L_t - L_s) dt_s (s <= t)
            dcb16 = torch.empty(n * G * Q, Q, dtype=dtp, device=dev)
            rc = NV.lib().fmsb_ssd_dcb(dG.data_ptr(), Lt[c0:c1].data_ptr(), dtt[c0:c1].data_ptr(), dcb16.data_ptr(), n,
                                       nh, G, Q, code, NV.stream_ptr())
            NV.check(rc, "fmsb_ssd_dcb")
            del dG
            dC[rows] += batched_gemm(dcb16, B2[rows], M=Q, N=N, K=Q, n_batch=n * G, n_inner=G, a_off=(G * Q, Q, 0, 1),
                                     b_off=(Q, 0, N, 1), d_off=(Q, 0, N), b_mn=True, out_rows=n * Q, out_cols=G * N,
                                     out_dtype=torch.float32)
            dB[rows] += batched_gemm(dcb16, C2[rows], M=Q, N=N, K=Q, n_batch=n * G, n_inner=G, a_off=(G * Q, Q, 0, 1),
                                     b_off=(Q, 0, N, 1), d_off=(Q, 0, N), a_mn=True, b_mn=True, out_rows=n * Q,
                                     out_cols=G * N, out_dtype=torch.float32)
            del dcb16
        # ---- dx and the per-(t, h) dot products, one pass over the [T, heads, P] tensors
        dx = torch.empty(T, nh, P, dtype=dtp, device=dev)
        red = torch.empty(5, T, nh, dtype=torch.float32, device=dev)
        Df = D.float().contiguous()
        rc = NV.lib().fmsb_ssd_bwd_combine(dy2.data_ptr(), x2.data_ptr(), y_inter.data_ptr(), dxw.data_ptr(),
                                           dx_intra.data_ptr(), y_intra.data_ptr(), L.data_ptr(), wgt.data_ptr(),
                                           Df.data_ptr(), dx.data_ptr(), red.data_ptr(), T * nh, P, nh, code,
                                           NV.stream_ptr())
        NV.check(rc, "fmsb_ssd_bwd_combine")
        del y_inter, dxw, dx_intra, y_intra
        dD = red[0].sum(0)
        dww = red[2] * wgt                                                    # through w = exp(Ltot - L) dt
        row, col = red[3], red[4]                                             # sums of dG o G over s / over t
        dL = red[1] - dww + row - col
        ddt = (dww + col) / dt
        dLtot = dLtot + dww.view(nc, Q, nh).sum(1)
        # ---- through L = cumsum(dt A) within the chunk, Ltot = L[last]: a reverse cumulative sum per chunk
        dLt = _chunk_major(dL, nc, Q, nh)
        dLt[:, :, -1] += dLtot
        dat = dLt.sum(-1, keepdim=True) - dLt.cumsum(-1) + dLt
        da = dat.transpose(1, 2).reshape(T, nh)
        ddt = ddt + da * A.float()[None, :]
        dA = (da * dt).sum(0)
        return (dx, ddt.to(dt.dtype), dA.to(A.dtype), dB.view(T, G, N).to(B.dtype), dC.view(T, G, N).to(C.dtype),
                dD.to(D.dtype), dh0, None, None, None)


class _StateCorrection(torch.autograd.Function):
    """y = y0 + exp(Lg) (C . H_in): what a state ``H_in [nh, P, N]`` entering the slice adds to the outputs of a
    zero-initial-state scan ``y0 [T, nh, P]``, with ``Lg`` the cumulative ``dt*A`` from the start of the slice."""

    @staticmethod
    def forward(ctx, y0, h_in, dt, A, C, Q):
        T, nh, P = y0.shape
        G, N = C.shape[1], C.shape[2]
        nc, hpg = T // Q, nh // G
        dtp = y0.dtype
        dt = dt.float().contiguous()
        Lg = (dt * A.float()[None, :]).t().contiguous().cumsum(-1).t().contiguous()   # [T, nh]
        hin16 = h_in.to(dtp).reshape(nh * P, N).contiguous()
        C2 = C.reshape(T, G * N)
        yc = _state_gemm(C2, hin16, T, Q, nh, P, N, hpg)
        y02 = _rows16(y0.reshape(T, nh * P))
        y = torch.empty(T, nh, P, dtype=dtp, device=y0.device)
        rc = NV.lib().fmsb_ssd_addscaled(y02.data_ptr(), yc.data_ptr(), Lg.data_ptr(), y.data_ptr(), T * nh, P,
                                         NV.dtype_code(dtp), NV.stream_ptr())
        NV.check(rc, "fmsb_ssd_addscaled")
        ctx.save_for_backward(hin16, dt, A, C, Lg)
        ctx.meta = (Q, h_in.dtype)
        return y

    @staticmethod
    def backward(ctx, dy):
        hin16, dt, A, C, Lg = ctx.saved_tensors
        Q, h_dtype = ctx.meta
        T, nh, P = dy.shape
        G, N = C.shape[1], C.shape[2]
        nc, hpg = T // Q, nh // G
        dtp = dy.dtype
        code = NV.dtype_code(dtp)
        C2 = C.reshape(T, G * N)
        dy2 = _rows16(dy.reshape(T, nh * P))
        dyi = _rowscale(dy2, torch.exp(Lg), nh, P)
        # dC[c, g] [Q, N] = dyi[c, heads of g] [Q, hpg*P] . H_in[heads of g] [(h,p), N]
        dC = batched_gemm(dyi, hin16, M=Q, N=N, K=hpg * P, n_batch=nc * G, n_inner=G, a_off=(Q, 0, hpg * P, 1),
                          b_off=(0, hpg * P, 0, 1), d_off=(Q, 0, N), b_mn=True, out_rows=T, out_cols=G * N,
                          out_dtype=torch.float32)
        # dH_in[h] [P, N] = dyi[:, h]^T C  (contraction over the T rows of the slice)
        dh = batched_gemm(dyi, C2, M=P, N=N, K=T, n_batch=nh, n_inner=nh, a_off=(0, 0, P, 1), b_off=(0, 0, N, hpg),
                          d_off=(0, P, 0), a_mn=True, b_mn=True, out_rows=nh * P, out_cols=N, out_dtype=torch.float32)
        del dyi
        # dLg[t, h] = exp(Lg) dy[t, h, :] . (C_t . H_in[h])
        yc = _state_gemm(C2, hin16, T, Q, nh, P, N, hpg)
        dLg = torch.empty(T, nh, dtype=torch.float32, device=dy.device)
        rc = NV.lib().fmsb_ssd_rowdot(dy2.data_ptr(), yc.data_ptr(), Lg.data_ptr(), dLg.data_ptr(), T * nh, P, code,
                                      NV.stream_ptr())
        NV.check(rc, "fmsb_ssd_rowdot")
        del yc
        dLgt = dLg.t().contiguous()                                           # through Lg = cumsum(dt A)
        da = (dLgt.sum(-1, keepdim=True) - dLgt.cumsum(-1) + dLgt).t()
        ddt = da * A.float()[None, :]
        dA = (da * dt).sum(0)
        return dy, dh.view(nh, P, N).to(h_dtype), ddt, dA.to(A.dtype), dC.view(T, G, N).to(C.dtype), None


def _state_gemm(C2, hin16, T, Q, nh, P, N, hpg):
    """[T, nh*P] fp32: row t, head h = C_t . H_in[h]^T, as nc*nh products of [Q, N] x [N, P] on tcgen05."""
    nc = T // Q
    return batched_gemm(C2, hin16, M=Q, N=P, K=N, n_batch=nc * nh, n_inner=nh, a_off=(Q, 0, N, hpg),
                        b_off=(0, P, 0, 1), d_off=(Q, 0, P), out_rows=T, out_cols=nh * P, out_dtype=torch.float32)


def state_correction_ref(y0, h_in, dt, A, C):
    """PyTorch statement of :class:`_StateCorrection` (oracle)."""
    T, nh, P = y0.shape
    G = C.shape[1]
    Lg = torch.cumsum(dt.float() * A.float()[None, :], 0)
    Ch = C.float().repeat_interleave(nh // G, 1)
    return y0.float() + torch.exp(Lg)[:, :, None] * torch.einsum("thn,hpn->thp", Ch, h_in.float())


def state_correction(y0, h_in, dt, A, C, chunk_size=256):
    """Add the contribution of the state entering the slice to a zero-initial-state scan output."""
    if not y0.is_cuda:
        return state_correction_ref(y0, h_in, dt, A, C).to(y0.dtype)
    return _StateCorrection.apply(y0, h_in, dt, A, C, chunk_size)


def ssd_scan(x, dt, A, B, C, D, h0=None, chunk_size=256, recompute=False, cp=None):
    """Chunked SSD scan.  Returns ``(y [T, nh, P], final_state [nh, P, N] fp32)``.  ``recompute``: keep only the
    inputs for the backward, which rebuilds the per-chunk entering states (the ``mamba_recompute`` switch of the
    context-parallel plugin, fms_acceleration_mcp/framework_plugin_mcp.py:37-44)."""
    if not x.is_cuda:
        y, h = ssd_ref(x, dt, A, B, C, D, h0)
        return y.to(x.dtype), h.float()
    return _SSDScan.apply(x, dt, A, B, C, D, h0, chunk_size, bool(recompute), cp)
