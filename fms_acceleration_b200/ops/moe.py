"""Mixture-of-experts execution: router, device-side plan, dispatch, grouped tcgen05 GEMMs, combine
(``csrc/moe.cu`` and the grouped modes of ``csrc/gemm_tcgen05.cu``).

Same math as the reference's ScatterMoE path (fms_acceleration_moe/utils/scattermoe.py:411-491,
scattermoe_utils/khd/kernels/ops/__init__.py:59-278, scattermoe_utils/expert_parallel.py:97-232):
``out[t] = sum_k gate[t,k] * W2[e] (act(W1[e] x_t) * W3[e] x_t)`` with ``e = topk(t, k)``, expert weights stored
``[E, in, out]``.  With expert parallelism every rank owns ``E / ep`` experts; rows travel to the owner by peer
stores and results come back by peer loads, two device-side barriers per layer and direction, no host sync.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import os

import torch
import torch.distributed as dist

from .. import _native as N
from . import activation as ACT

P, I, L, F, U = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_uint
N.declare("fmsb_grouped_gemm", [P, L, P, L, I, I, P, L, I, P, L, F, F, I, I, I, I, I, I, P, L, L, L, P, P])
N.declare("fmsb_moe_router", [P, I, I, I, I, P, P, P])
N.declare("fmsb_moe_router_bwd", [P, P, P, P, I, I, I, I, P, P])
N.declare("fmsb_moe_plan", [P, L, I, I, I, I, P, P, P, U, P, P, P, P, P, P, P, P])
N.declare("fmsb_moe_dispatch", [P, L, P, P, P, L, I, I, I, P, L, I, I, P])
N.declare("fmsb_moe_zero_pad", [P, L, I, P, P, I, I, P])
N.declare("fmsb_moe_combine", [P, L, P, P, P, L, I, I, I, P, L, I, I, P])
N.declare("fmsb_moe_gate_grad", [P, L, P, P, P, L, L, I, I, I, P, I, I, P])
N.declare("fmsb_moe_dispatch_meta", [P, L, P, P, P, L, I, I, I, P, L, P, I, I, P])
N.declare("fmsb_moe_rowdot_scale", [P, L, P, L, P, P, P, I, I, I, I, P])
N.declare("fmsb_moe_gather_scalar", [P, P, P, L, I, P, I, P])


# ------------------------------------------------------------------------------------------------ oracle
def moe_ref(x, router_w, w1, w2, w3, top_k, act="silu", renorm=True, idx=None):
    """Dense fp32 oracle.  x [T,H]; router_w [E,H]; w1,w3 [E,H,I]; w2 [E,I,H].  ``idx`` ([T,k]) fixes the routing
    decisions (near-ties may otherwise be broken differently by a lower-precision router)."""
    xf = x.float()
    logits = xf @ router_w.float().t()
    probs = torch.softmax(logits, dim=-1)
    if idx is None:
        w, idx = torch.topk(probs, top_k, dim=-1)
    else:
        idx = idx.long()
        w = torch.gather(probs, 1, idx)
    if renorm:
        w = w / w.sum(-1, keepdim=True)
    out = torch.zeros_like(xf)
    fn = {"silu": torch.nn.functional.silu, "gelu": torch.nn.functional.gelu}.get(act, torch.nn.functional.silu)
    for e in range(w1.shape[0]):
        tok, slot = torch.nonzero(idx == e, as_tuple=True)
        if tok.numel() == 0:
            continue
        xe = xf[tok]
        h = fn(xe @ w1[e].float()) * (xe @ w3[e].float())
        out.index_add_(0, tok, (h @ w2[e].float()) * w[tok, slot][:, None])
    return out, logits


# ------------------------------------------------------------------------------------------------ kernels
def grouped_gemm(a, b, seg_off, n_groups, *, mode, b_mn=True, out=None, out_dtype=None, c=None, beta=0.0, n=None, m=None):
    """mode 1: out[rows, n] = a[rows, K] @ B_g per segment; b [E*in, out] viewed 2-D.
    mode 2: out[g] = a[seg_g]^T @ b[seg_g]  -> out [n_groups, m, n]."""
    st = N.status_word(a.device)
    fmt = N.dtype_code(a.dtype)
    if mode == 1:
        rows, K = a.shape
        if out is None:
            out = torch.empty(rows, n, dtype=out_dtype or a.dtype, device=a.device)
        bn = 256 if n >= 192 else (128 if n > 64 else 64)
        rc = N.lib().fmsb_grouped_gemm(a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0), K, int(b_mn), out.data_ptr(),
                                       out.stride(0), int(out.dtype == torch.float32), N.ptr(c),
                                       c.stride(0) if c is not None else 0, 1.0, float(beta), 0, n, fmt, bn, 1, n_groups,
                                       seg_off.data_ptr(), 0, rows, b.shape[0], st.data_ptr(), N.stream_ptr())
    else:
        if out is None:
            out = torch.empty(n_groups, m, n, dtype=out_dtype or torch.float32, device=a.device)
        bn = 256 if n >= 192 else (128 if n > 64 else 64)
        rc = N.lib().fmsb_grouped_gemm(a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0), 64, 1, out.data_ptr(),
                                       out.stride(1), int(out.dtype == torch.float32), None, 0, 1.0, 0.0, m, n, fmt, bn, 2,
                                       n_groups, seg_off.data_ptr(), out.stride(0), a.shape[0], b.shape[0], st.data_ptr(),
                                       N.stream_ptr())
    N.check(rc, "fmsb_grouped_gemm")
    return out


class _RouterTopK(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, k, renorm):
        lg = logits.float().contiguous()
        T, E = lg.shape
        idx = torch.empty(T, k, dtype=torch.int32, device=lg.device)
        w = torch.empty(T, k, dtype=torch.float32, device=lg.device)
        rc = N.lib().fmsb_moe_router(lg.data_ptr(), T, E, k, int(renorm), idx.data_ptr(), w.data_ptr(), N.stream_ptr())
        N.check(rc, "fmsb_moe_router")
        ctx.save_for_backward(lg, idx, w)
        ctx.meta = (k, renorm, logits.dtype)
        ctx.mark_non_differentiable(idx)
        return w, idx

    @staticmethod
    def backward(ctx, dw, _didx):
        lg, idx, w = ctx.saved_tensors
        k, renorm, dt = ctx.meta
        T, E = lg.shape
        dlog = torch.empty_like(lg)
        rc = N.lib().fmsb_moe_router_bwd(lg.data_ptr(), idx.data_ptr(), w.data_ptr(), dw.float().contiguous().data_ptr(),
                                         T, E, k, int(renorm), dlog.data_ptr(), N.stream_ptr())
        N.check(rc, "fmsb_moe_router_bwd")
        return dlog.to(dt), None, None


def router_topk(logits, k, renorm=True):
    """(weights fp32 [T,k], indices int32 [T,k]) of the top-k experts by softmax probability."""
    if not logits.is_cuda:
        p = torch.softmax(logits.float(), dim=-1)
        w, idx = torch.topk(p, k, dim=-1)
        if renorm:
            w = w / w.sum(-1, keepdim=True)
        return w, idx.to(torch.int32)
    return _RouterTopK.apply(logits, k, renorm)


class MoEContext:
    """Per-layer buffers and the communication state of one mixture-of-experts layer."""

    _shared: dict = {}

    def __init__(self, hidden: int, inter: int, num_experts: int, top_k: int, group=None,
                 capacity_factor: Optional[float] = None, layer_tag: str = "moe"):
        if capacity_factor is None:
            capacity_factor = float(os.environ.get("FMSB_MOE_CAPACITY_FACTOR", "2.0"))
        self.H, self.I, self.E, self.k = hidden, inter, num_experts, top_k
        self.group = group
        self.world = dist.get_world_size(group) if (group is not None and dist.is_initialized()) else 1
        self.rank = dist.get_rank(group) if self.world > 1 else 0
        self.E_local = num_experts // self.world
        self.capacity_factor = capacity_factor
        self.tag = layer_tag
        self.cap = 0
        self.comm = None
        self._bufs = {}

    # symmetric (world > 1) or plain buffers
    def _alloc(self, key, rows, cols, dtype, device, shared=False):
        store = MoEContext._shared if shared else self._bufs
        k = (key, rows, cols, dtype, self.world, id(self.group) if shared else 0)
        ent = store.get(k)
        if ent is None:
            nbytes = rows * cols * torch.empty((), dtype=dtype).element_size()
            if self.world > 1:
                from ..parallel.symm import SymmBuffer

                sb = SymmBuffer(nbytes, self.group, device, zero=True)
                t = sb.view(0, rows * cols, dtype).view(rows, cols)
                ent = (t, sb.ptr_array(), sb)
            else:
                t = torch.zeros(rows, cols, dtype=dtype, device=device)
                ent = (t, (ctypes.c_void_p * 1)(t.data_ptr()), None)
            store[k] = ent
        return ent

    def ensure(self, T: int, dtype, device):
        if self.world == 1:
            rows = T * self.k  # exact upper bound: the local buffer can never overflow
        else:
            # T*k rows arrive per rank when routing is balanced, world*T*k when every token of every rank picks this
            # rank's experts; rows beyond the capacity are dropped and reported (status 7), never written
            rows = int(min(self.capacity_factor, float(self.world)) * T * self.k)
        cap = (rows + self.E_local * 128 + 127) // 128 * 128
        if cap != self.cap:
            self.cap = cap
        if self.world > 1 and self.comm is None:
            key = ("comm", id(self.group))
            if key not in MoEContext._shared:
                from ..parallel.symm import Communicator, SymmBuffer

                comm = Communicator(self.group, device)
                tables = SymmBuffer(2 * self.world * self.E * 4, self.group, device)
                MoEContext._shared[key] = (comm, tables)
            self.comm, self.tables = MoEContext._shared[key]
        return cap

    def barrier(self, chan):
        if self.world > 1:
            self.comm.barrier(chan)

    # rows an owner would have needed so far for nothing to be dropped (maximum over layers, steps and owners)
    _needed: dict = {}

    @classmethod
    def needed_counter(cls, device) -> torch.Tensor:
        dev = torch.device(device)
        key = dev.index if dev.index is not None else torch.cuda.current_device()
        t = cls._needed.get(key)
        if t is None:
            t = torch.zeros(1, dtype=torch.int32, device=f"cuda:{key}")
            cls._needed[key] = t
        return t

    @classmethod
    def max_rows_needed(cls, device=None) -> int:
        """Host-synchronising read of the counter; compare with ``T * top_k`` to choose ``capacity_factor``."""
        return int(cls.needed_counter(device if device is not None else torch.cuda.current_device()).item())


PLAN_CHAN = 8
BAR_A, BAR_B, BAR_C, BAR_D = 10, 11, 12, 13


def _plan(ctx: MoEContext, topk_idx, T, device):
    E, k = ctx.E, ctx.k
    counts = torch.zeros(E, dtype=torch.int32, device=device)
    seg_off = torch.empty(ctx.E_local + 1, dtype=torch.int32, device=device)
    seg_cnt = torch.empty(ctx.E_local, dtype=torch.int32, device=device)
    send_base = torch.empty(2 * E, dtype=torch.int32, device=device)  # [first slot | end of valid slots] per expert
    dest_row = torch.empty(T, k, dtype=torch.int32, device=device)
    scratch = torch.empty(max(1, -(-T * k // 1024)) * E, dtype=torch.int32, device=device)  # per-chunk expert counts
    st = N.status_word(device)
    if ctx.world > 1:
        epoch = ctx.comm.next_epoch(PLAN_CHAN)
        slot = epoch & 1
        tab = ctx.tables.ptr_array(slot * ctx.world * E * 4)
        sig = ctx.comm.signals.ptr_array(PLAN_CHAN * ctx.world * 4)
    else:
        epoch, tab, sig = 0, None, None
    rc = N.lib().fmsb_moe_plan(topk_idx.data_ptr(), T * k, E, ctx.rank, ctx.world, ctx.cap, counts.data_ptr(), tab, sig,
                               epoch, seg_off.data_ptr(), seg_cnt.data_ptr(), send_base.data_ptr(), dest_row.data_ptr(),
                               MoEContext.needed_counter(device).data_ptr(), scratch.data_ptr(), st.data_ptr(),
                               N.stream_ptr())
    N.check(rc, "fmsb_moe_plan")
    return seg_off, seg_cnt, dest_row


def _dispatch(ctx, x, topk_idx, dest_row, scale, buf_ptrs, ld):
    T = x.shape[0]
    rc = N.lib().fmsb_moe_dispatch(x.data_ptr(), x.stride(0), topk_idx.data_ptr(), dest_row.data_ptr(), N.ptr(scale),
                                   T * ctx.k, ctx.k, x.shape[1], ctx.E_local, buf_ptrs, ld, ctx.world,
                                   N.dtype_code(x.dtype), N.stream_ptr())
    N.check(rc, "fmsb_moe_dispatch")


def _zero_pad(ctx, buf, seg_off, seg_cnt):
    rc = N.lib().fmsb_moe_zero_pad(buf.data_ptr(), buf.stride(0), buf.shape[1], seg_off.data_ptr(), seg_cnt.data_ptr(),
                                   ctx.E_local, N.dtype_code(buf.dtype), N.stream_ptr())
    N.check(rc, "fmsb_moe_zero_pad")


def _combine(ctx, buf_ptrs, ld, topk_idx, dest_row, w, T, H, dtype, device):
    out = torch.empty(T, H, dtype=dtype, device=device)
    rc = N.lib().fmsb_moe_combine(buf_ptrs, ld, topk_idx.data_ptr(), dest_row.data_ptr(), N.ptr(w), T, ctx.k, H,
                                  ctx.E_local, out.data_ptr(), out.stride(0), ctx.world, N.dtype_code(dtype),
                                  N.stream_ptr())
    N.check(rc, "fmsb_moe_combine")
    return out


class _Experts(torch.autograd.Function):
    """x [T,H], gates fp32 [T,k], idx int32 [T,k], w1/w3 [E_local,H,I], w2 [E_local,I,H] -> [T,H]."""

    @staticmethod
    def forward(ctx, x, gates, idx, w1, w3, w2, mctx: MoEContext, act: str):
        T, H = x.shape
        I_, El = mctx.I, mctx.E_local
        dev, dt = x.device, x.dtype
        cap = mctx.ensure(T, dt, dev)
        seg_off, seg_cnt, dest_row = _plan(mctx, idx, T, dev)
        Xs, Xs_ptrs, _ = mctx._alloc("Xs", cap, H, dt, dev)
        Ys, Ys_ptrs, _ = mctx._alloc("Ys", cap, H, dt, dev)
        _zero_pad(mctx, Xs, seg_off, seg_cnt)
        _dispatch(mctx, x, idx, dest_row, None, Xs_ptrs, Xs.stride(0))
        mctx.barrier(BAR_A)
        gu = torch.empty(cap, 2 * I_, dtype=dt, device=dev)
        grouped_gemm(Xs, w1.view(El * H, I_), seg_off, El, mode=1, n=I_, out=gu[:, :I_])
        grouped_gemm(Xs, w3.view(El * H, I_), seg_off, El, mode=1, n=I_, out=gu[:, I_:])
        hs = ACT.glu_fwd(gu[:, :I_], gu[:, I_:], act)
        grouped_gemm(hs, w2.view(El * I_, H), seg_off, El, mode=1, n=H, out=Ys)
        mctx.barrier(BAR_B)
        out = _combine(mctx, Ys_ptrs, Ys.stride(0), idx, dest_row, gates, T, H, dt, dev)
        ctx.mctx, ctx.act = mctx, act
        ctx.save_for_backward(gates, idx, w1, w3, w2, seg_off, seg_cnt, dest_row, gu)
        return out

    @staticmethod
    def backward(ctx, dout):
        mctx, act = ctx.mctx, ctx.act
        gates, idx, w1, w3, w2, seg_off, seg_cnt, dest_row, gu = ctx.saved_tensors
        dout = dout.contiguous()
        T, H = dout.shape
        I_, El, cap = mctx.I, mctx.E_local, gu.shape[0]
        dev, dt = dout.device, dout.dtype
        Xs, Xs_ptrs, _ = mctx._alloc("Xs", cap, H, dt, dev)
        Ys, Ys_ptrs, _ = mctx._alloc("Ys", cap, H, dt, dev)
        dYs, dYs_ptrs, _ = mctx._alloc("dYs", cap, H, dt, dev, shared=True)
        dXs, dXs_ptrs, _ = mctx._alloc("dXs", cap, H, dt, dev, shared=True)
        # dout rows travel unscaled together with their routing weight; the OWNER forms <expert output, dout> per row
        # (the routing-weight gradient) and applies the weight, so only 4 bytes per pair come back instead of a second
        # pull of every expert-output row
        rgate, rgate_ptrs, _ = mctx._alloc("rgate", cap, 1, torch.float32, dev, shared=True)
        rdots, rdots_ptrs, _ = mctx._alloc("rdots", cap, 1, torch.float32, dev, shared=True)
        _zero_pad(mctx, dYs, seg_off, seg_cnt)
        gates_c = gates.contiguous()
        rc = N.lib().fmsb_moe_dispatch_meta(dout.data_ptr(), dout.stride(0), idx.data_ptr(), dest_row.data_ptr(),
                                            gates_c.data_ptr(), T * mctx.k, mctx.k, H, El, dYs_ptrs, dYs.stride(0),
                                            rgate_ptrs, mctx.world, N.dtype_code(dt), N.stream_ptr())
        N.check(rc, "fmsb_moe_dispatch_meta")
        mctx.barrier(BAR_C)
        rc = N.lib().fmsb_moe_rowdot_scale(Ys.data_ptr(), Ys.stride(0), dYs.data_ptr(), dYs.stride(0), rgate.data_ptr(),
                                           rdots.data_ptr(), seg_off.data_ptr(), El, cap, H, N.dtype_code(dt),
                                           N.stream_ptr())
        N.check(rc, "fmsb_moe_rowdot_scale")
        hs = ACT.glu_fwd(gu[:, :I_], gu[:, I_:], act)
        dw2 = grouped_gemm(hs, dYs, seg_off, El, mode=2, m=I_, n=H)
        dhs = grouped_gemm(dYs, w2.view(El * I_, H), seg_off, El, mode=1, b_mn=False, n=I_)
        ACT.glu_bwd(dhs, gu[:, :I_], gu[:, I_:], act, de=gu[:, :I_], dg=gu[:, I_:])
        dg1 = gu[:, :I_]
        dg3 = gu[:, I_:]
        dw1 = grouped_gemm(Xs, dg1, seg_off, El, mode=2, m=H, n=I_)
        dw3 = grouped_gemm(Xs, dg3, seg_off, El, mode=2, m=H, n=I_)
        grouped_gemm(dg1, w1.view(El * H, I_), seg_off, El, mode=1, b_mn=False, n=H, out=dXs)
        grouped_gemm(dg3, w3.view(El * H, I_), seg_off, El, mode=1, b_mn=False, n=H, out=dXs, c=dXs, beta=1.0)
        mctx.barrier(BAR_D)
        dx = _combine(mctx, dXs_ptrs, dXs.stride(0), idx, dest_row, None, T, H, dt, dev)
        dgate = torch.empty(T, mctx.k, dtype=torch.float32, device=dev)
        rc = N.lib().fmsb_moe_gather_scalar(rdots_ptrs, idx.data_ptr(), dest_row.data_ptr(), T * mctx.k, El,
                                            dgate.data_ptr(), mctx.world, N.stream_ptr())
        N.check(rc, "fmsb_moe_gather_scalar")
        return dx, dgate, None, dw1.to(w1.dtype), dw3.to(w3.dtype), dw2.to(w2.dtype), None, None


def experts_forward(x, gates, idx, w1, w3, w2, mctx: MoEContext, act="silu"):
    return _Experts.apply(x, gates, idx, w1, w3, w2, mctx, act)
