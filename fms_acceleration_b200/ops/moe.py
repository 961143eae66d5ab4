"""Mixture-of-experts execution: router, device-side plan, dispatch, grouped tcgen05 GEMMs, combine
(``csrc/moe.cu`` and the grouped modes of ``csrc/gemm_tcgen05.cu``).

Same math as the reference's ScatterMoE path (fms_acceleration_moe/utils/scattermoe.py:411-491,
scattermoe_utils/khd/kernels/ops/__init__.py:59-278, scattermoe_utils/expert_parallel.py:97-232):
``out[t] = sum_k gate[t,k] * W2[e] (act(W1[e] x_t) * W3[e] x_t)`` with ``e = topk(t, k)``, expert weights stored
``[E, in, out]``.  Gate and up projection run as one grouped GEMM over the two weight tensors side by side, and so
do their weight gradients and the input gradient through both.

Expert parallelism (every rank owns ``E / ep`` experts), no host synchronisation anywhere:

* **One row per (token, destination rank).**  A token whose experts live on ``r`` ranks crosses NVLink ``r`` times
  instead of ``top_k`` times: the source stores the row once into each destination's staging block together with
  the slots it must be replicated to and its routing weights; the owner replicates locally into its expert-sorted
  buffer, and on the way back sums the (weighted) expert outputs of a staged row into one row that the source
  pulls.  For 40 experts on 8 ranks with top-8 that is 5.6 instead of 8 rows per token and direction, on 2 ranks
  2 instead of 8.
* **Token chunks pipelined over two streams (optional).**  The tokens of a call can be cut into ``n_chunks`` slices;
  dispatch and combine of one slice then run on a communication stream while the grouped GEMMs of the neighbouring
  slice run on the compute stream (two staging sets, reused every other chunk; the cross-rank barriers that order
  the reuse are on the communication stream).  One slice is the default: see :class:`MoEContext`.
* **Fixed layout from an agreed token budget.**  Staging blocks and the expert-sorted capacity are sized once from
  the largest number of tokens a rank may bring to one call (agreed over the group at set-up), so ranks whose
  padding-free batches differ in length still address the same layout and nothing is re-allocated per step.  Rows
  beyond the capacity are dropped on every rank alike and counted (:func:`overflow_count`), never written.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch
import torch.distributed as dist

from .. import _native as N
from . import activation as ACT

P, I, L, F, U = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_uint
N.declare("fmsb_grouped_gemm", [P, L, P, L, I, I, P, L, I, P, L, F, F, I, I, I, I, I, I, P, L, L, L, P, P])
N.declare("fmsb_grouped_gemm2", [P, L, P, L, I, I, P, I, P, L, P, L, I, P, L, I, P, L, I, F, F, I, I, I, I, I, I, P, L,
                                 L, L, I, P, P])
N.declare("fmsb_moe_router", [P, I, I, I, I, P, P, P])
N.declare("fmsb_moe_router_bwd", [P, P, P, P, I, I, I, I, P, P])
N.declare("fmsb_moe_plan", [P, L, I, I, I, I, P, P, P, U, P, P, P, P, P, P, P, P, P])
N.declare("fmsb_moe_dispatch", [P, L, P, P, P, L, I, I, I, P, L, I, I, P])
N.declare("fmsb_moe_zero_pad", [P, L, I, P, P, I, I, P])
N.declare("fmsb_moe_combine", [P, L, P, P, P, L, I, I, I, P, L, I, I, P])
N.declare("fmsb_moe_gate_grad", [P, L, P, P, P, L, L, I, I, I, P, I, I, P])
N.declare("fmsb_moe_dispatch_meta", [P, L, P, P, P, L, I, I, I, P, L, P, I, I, P])
N.declare("fmsb_moe_rowdot_scale", [P, L, P, L, P, P, P, I, I, I, I, P])
N.declare("fmsb_moe_gather_scalar", [P, P, P, L, I, P, I, P])
N.declare("fmsb_moe_stage_plan", [P, P, L, I, I, I, P, P, P, P, P, P])
N.declare("fmsb_moe_dispatch_staged", [P, L, P, P, P, P, P, L, I, I, I, I, I, P, L, P, P, P, I, P])
N.declare("fmsb_moe_replicate", [P, L, P, P, P, L, I, P, I, I, P, L, I, P])
N.declare("fmsb_moe_prereduce", [P, L, P, P, L, I, P, I, I, P, L, I, P])


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
def _bn(n: int) -> int:
    return 256 if n >= 192 else (128 if n > 64 else 64)


def grouped_gemm(a, b, seg_off, n_groups, *, mode, b_mn=True, out=None, out_dtype=None, c=None, beta=0.0, n=None, m=None,
                 b_alt=None, a2=None, b2=None, max_ctas=0):
    """mode 1: out[rows, n] = a[rows, K] @ B_g per segment; b [E*in, out] viewed 2-D.  ``b_alt``: a second weight
    tensor of the same shape whose product fills the right half of ``out`` (n = 2 * b.shape[1]).  ``a2``/``b2``: a
    second operand pair accumulated into the same tile (``out = a @ B_g + a2 @ B2_g``).
    mode 2: out[g] = a[seg_g]^T @ b[seg_g]  -> out [n_groups, m, n]; ``c`` (fp32, = out) with ``beta=1`` accumulates."""
    st = N.status_word(a.device)
    fmt = N.dtype_code(a.dtype)
    if mode == 1:
        rows, K = a.shape
        if out is None:
            out = torch.empty(rows, n, dtype=out_dtype or a.dtype, device=a.device)
        n_split = b.shape[1] if b_alt is not None else 0
        bn = _bn(n_split if n_split else n)
        if n_split and n_split % bn:
            bn = 128 if n_split % 128 == 0 else 64
        K2 = a2.shape[1] if a2 is not None else 0
        rc = N.lib().fmsb_grouped_gemm2(a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0), K, int(b_mn), N.ptr(b_alt),
                                        n_split, N.ptr(a2), a2.stride(0) if a2 is not None else 0, N.ptr(b2),
                                        b2.stride(0) if b2 is not None else 0, K2, out.data_ptr(), out.stride(0),
                                        int(out.dtype == torch.float32), N.ptr(c), c.stride(0) if c is not None else 0,
                                        int(c is not None and c.dtype == torch.float32), 1.0, float(beta), 0, n, fmt, bn,
                                        1, n_groups, seg_off.data_ptr(), 0, rows, b.shape[0], int(max_ctas),
                                        st.data_ptr(), N.stream_ptr())
    else:
        if out is None:
            out = torch.empty(n_groups, m, n, dtype=out_dtype or torch.float32, device=a.device)
        rc = N.lib().fmsb_grouped_gemm2(a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0), 64, 1, None, 0, None, 0,
                                        None, 0, 0, out.data_ptr(), out.stride(1), int(out.dtype == torch.float32),
                                        N.ptr(c), c.stride(1) if c is not None else 0,
                                        int(c is not None and c.dtype == torch.float32), 1.0, float(beta), m, n, fmt,
                                        _bn(n), 2, n_groups, seg_off.data_ptr(), out.stride(0), a.shape[0], b.shape[0],
                                        int(max_ctas), st.data_ptr(), N.stream_ptr())
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


# ------------------------------------------------------------------------------------------------ state
_overflow: dict = {}
_needed: dict = {}


def _dev_index(device) -> int:
    dev = torch.device(device) if device is not None else None
    return dev.index if dev is not None and dev.index is not None else torch.cuda.current_device()


def _counter(store: dict, device) -> torch.Tensor:
    key = _dev_index(device)
    t = store.get(key)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=f"cuda:{key}")
        store[key] = t
    return t


def overflow_count(device=None, reset: bool = False) -> int:
    """Host-synchronising read of the number of experts (summed over calls) whose rows did not all fit into an
    owner's receive capacity, i.e. whose excess rows were dropped.  Informational: training continues."""
    t = _counter(_overflow, device)
    v = int(t.item())
    if reset:
        t.zero_()
    return v


def _round_up(n: int, a: int) -> int:
    return (n + a - 1) // a * a


class _EPShared:
    """What all mixture-of-experts layers of one expert-parallel group share: the communicator, the histogram
    tables of the plan, and two sets of staging buffers.  Allocated ONCE (one symmetric allocation, one
    rendezvous), sized from the agreed token budget."""

    def __init__(self, group, device, dtype, H: int, k: int, E: int, token_budget: int, n_chunks: int,
                 capacity_factor: float):
        from ..parallel.symm import Communicator, SymmBuffer

        self.group, self.device, self.dtype = group, device, dtype
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.H, self.k, self.E = H, k, E
        self.E_local = E // self.world
        # the budget must be the same everywhere: take the largest one any rank asks for
        t = torch.tensor([int(token_budget), int(n_chunks)], dtype=torch.int64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
        self.token_budget, self.C = int(t[0]), max(1, int(t[1]))
        self.Tbc = _round_up(-(-self.token_budget // self.C), 8)  # staging rows per source rank and chunk
        self.cap = _round_up(int(min(capacity_factor, float(self.world)) * self.Tbc * k), 128) + self.E_local * 128
        self.comm = Communicator(group, device)
        self.stream = torch.cuda.Stream(device, priority=-1)
        esize = torch.empty((), dtype=dtype).element_size()
        rows = self.world * self.Tbc
        lay, off = {}, 0
        for s in range(2):
            for name, nbytes in (("x", rows * H * esize), ("y", rows * H * esize), ("slot", rows * k * 4),
                                 ("gate", rows * k * 4), ("cnt", 64 * 4), ("rdots", self.cap * 4)):
                lay[(name, s)] = off
                off = _round_up(off + nbytes, 256)
        lay["tables"] = off
        off = _round_up(off + 2 * self.world * E * 4, 256)
        self.buf = SymmBuffer(off, group, device, zero=True)
        self.off = lay
        self.ptrs = {key: self.buf.ptr_array(o) for key, o in lay.items()}
        self.stage_base = torch.tensor([self.rank * self.Tbc] * self.world + [(self.rank + 1) * self.Tbc] * self.world,
                                       dtype=torch.int32, device=device)
        torch.cuda.synchronize(device)
        dist.barrier(group)

    def local(self, name: str, s: int, dtype, rows: int, cols: int) -> torch.Tensor:
        return self.buf.view(self.off[(name, s)], rows * cols, dtype).view(rows, cols)

    def local_ptr(self, name: str, s: int) -> int:
        return self.buf.local.data_ptr() + self.off[(name, s)]

    def table_ptrs(self, slot: int):
        return self.buf.ptr_array(self.off["tables"] + slot * self.world * self.E * 4)


class MoEContext:
    """Geometry and communication state of one mixture-of-experts layer.

    ``token_budget``: the largest number of tokens this rank may hand to one call (expert parallelism only; default
    ``FMSB_MOE_TOKEN_BUDGET`` or, failing that, the maximum over the ranks of the first call's token count).
    ``n_chunks``: slices a call is pipelined in (``FMSB_MOE_CHUNKS``; default 1: on 4 and 8 GPUs the Granite step
    measured the same or slightly faster unsliced, 231.9 against 234.6 ms and 268.7 against 270.6 ms, because half-size
    grouped GEMMs and the doubled barriers cost what the overlap gains).  ``capacity_factor`` (default
    ``FMSB_MOE_CAPACITY_FACTOR`` or 2.0): receive capacity of an owner in units of the balanced load."""

    _shared: dict = {}

    def __init__(self, hidden: int, inter: int, num_experts: int, top_k: int, group=None,
                 capacity_factor: Optional[float] = None, layer_tag: str = "moe", token_budget: Optional[int] = None,
                 n_chunks: Optional[int] = None):
        if capacity_factor is None:
            capacity_factor = float(os.environ.get("FMSB_MOE_CAPACITY_FACTOR", "2.0"))
        self.H, self.I, self.E, self.k = hidden, inter, num_experts, top_k
        self.group = group
        self.world = dist.get_world_size(group) if (group is not None and dist.is_initialized()) else 1
        self.rank = dist.get_rank(group) if self.world > 1 else 0
        self.E_local = num_experts // self.world
        self.capacity_factor = capacity_factor
        self.token_budget = token_budget or int(os.environ.get("FMSB_MOE_TOKEN_BUDGET", "0")) or None
        # measured on two B200s (Granite-3B-sized layer): with one peer the exchange is small next to the fixed cost of a
        # second slice, so pipelining starts at four ranks
        self.n_chunks = n_chunks or int(os.environ.get("FMSB_MOE_CHUNKS", "0")) or 1
        self.gemm_ctas = int(os.environ.get("FMSB_MOE_GEMM_CTAS", "0"))  # 0: every SM
        self.tag = layer_tag
        self.cap = 0  # world == 1: rows of the expert-sorted buffer (tests may lower it to provoke an overflow)
        self.shared: Optional[_EPShared] = None

    def ensure_shared(self, T: int, dtype, device) -> _EPShared:
        if self.shared is None:
            key = (id(self.group), self.H, self.k, self.E, dtype)
            sh = MoEContext._shared.get(key)
            if sh is None:
                sh = _EPShared(self.group, device, dtype, self.H, self.k, self.E, self.token_budget or T, self.n_chunks,
                               self.capacity_factor)
                MoEContext._shared[key] = sh
            self.shared = sh
        if T > self.shared.token_budget:
            raise RuntimeError(
                f"{T} tokens in one mixture-of-experts call exceed the token budget {self.shared.token_budget} that the "
                "expert-parallel buffers were sized for; set FMSB_MOE_TOKEN_BUDGET (or token_budget=) to the largest "
                "per-rank token count of a step (per-device batch size x maximum sequence length)")
        return self.shared

    @classmethod
    def needed_counter(cls, device) -> torch.Tensor:
        return _counter(_needed, device)

    @classmethod
    def max_rows_needed(cls, device=None) -> int:
        """Host-synchronising read of the rows the busiest owner would have needed so far for nothing to be dropped
        (maximum over layers, steps, chunks and owners); compare with tokens-per-chunk x top_k to choose
        ``capacity_factor``."""
        return int(cls.needed_counter(device if device is not None else torch.cuda.current_device()).item())


PLAN_CHAN = 8
BAR_A, BAR_B, BAR_C, BAR_D = 10, 11, 12, 13


def _plan(ctx: MoEContext, topk_idx, T, device, cap=None):
    """Expert histogram -> (exchange over the group) -> segment layout of my experts and the slot of every pair."""
    E, k = ctx.E, ctx.k
    cap = ctx.cap if cap is None else cap
    counts = torch.zeros(E, dtype=torch.int32, device=device)
    seg_off = torch.empty(ctx.E_local + 1, dtype=torch.int32, device=device)
    seg_cnt = torch.empty(ctx.E_local, dtype=torch.int32, device=device)
    send_base = torch.empty(2 * E, dtype=torch.int32, device=device)  # [first slot | end of valid slots] per expert
    dest_row = torch.empty(T, k, dtype=torch.int32, device=device)
    scratch = torch.empty(max(1, -(-T * k // 1024)) * E, dtype=torch.int32, device=device)  # per-chunk expert counts
    st = N.status_word(device)
    if ctx.world > 1:
        sh = ctx.shared
        epoch = sh.comm.next_epoch(PLAN_CHAN)
        tab = sh.table_ptrs(epoch & 1)
        sig = sh.comm.signals.ptr_array(PLAN_CHAN * ctx.world * 4)
    else:
        epoch, tab, sig = 0, None, None
    rc = N.lib().fmsb_moe_plan(N.ptr(topk_idx) if T else None, T * k, E, ctx.rank, ctx.world, cap, counts.data_ptr(),
                               tab, sig, epoch, seg_off.data_ptr(), seg_cnt.data_ptr(), send_base.data_ptr(),
                               dest_row.data_ptr() if T else None, MoEContext.needed_counter(device).data_ptr(),
                               scratch.data_ptr(), _counter(_overflow, device).data_ptr(), st.data_ptr(),
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


def _combine(ctx, buf_ptrs, ld, topk_idx, dest_row, w, T, H, dtype, device, out=None, k=None, e_local=None, world=None):
    if out is None:
        out = torch.empty(T, H, dtype=dtype, device=device)
    if T == 0:
        return out
    rc = N.lib().fmsb_moe_combine(buf_ptrs, ld, topk_idx.data_ptr(), dest_row.data_ptr(), N.ptr(w), T,
                                  ctx.k if k is None else k, H, ctx.E_local if e_local is None else e_local,
                                  out.data_ptr(), out.stride(0), ctx.world if world is None else world,
                                  N.dtype_code(dtype), N.stream_ptr())
    N.check(rc, "fmsb_moe_combine")
    return out


def _one_ptr(t):
    return (ctypes.c_void_p * 1)(t.data_ptr())


# ------------------------------------------------------------------------------------------------ expert math
def _acc_gemm(acc, key, a, b, seg_off, n_groups, m, n, max_ctas):
    """Per-group ``a^T b`` into ``acc[key]`` (fp32): the first token slice writes it, later slices add to it."""
    if key not in acc:
        acc[key] = grouped_gemm(a, b, seg_off, n_groups, mode=2, m=m, n=n, max_ctas=max_ctas)
    else:
        grouped_gemm(a, b, seg_off, n_groups, mode=2, m=m, n=n, out=acc[key], c=acc[key], beta=1.0, max_ctas=max_ctas)


def _experts_fwd_local(mctx, Xs, seg_off, w1, w3, w2, act, Ys=None, lora=None):
    """gate|up (one grouped GEMM over the two weight tensors), activation, down projection.

    ``lora`` = (A13 [El, H, R13], B13 [El, R13, 2I], A2 [El, I, R2], B2 [El, R2, H]): per-expert low-rank factors,
    gate and up side by side in A13 and block-diagonal in B13.  Each projection is then
    ``rows . W_e + (rows . A_e) . B_e`` with the low-rank product accumulated into the same output tile as the
    frozen weight's (the second operand pair of the grouped kernel), never a dense ``W + A B`` per expert.  What
    the reference does in one Triton kernel (scattermoe_utils/khd/kernels/kernels.py:110-300)."""
    I_, El, H = mctx.I, mctx.E_local, mctx.H
    used = seg_off[El:]  # rows in use (device scalar): the buffers are sized for the capacity, not for the load
    if lora is None:
        gu = grouped_gemm(Xs, w1.view(El * H, I_), seg_off, El, mode=1, n=2 * I_, b_alt=w3.view(El * H, I_),
                          max_ctas=mctx.gemm_ctas)
        hs = ACT.glu_fwd(gu[:, :I_], gu[:, I_:], act, rows_dev=used)
        Ys = grouped_gemm(hs, w2.view(El * I_, H), seg_off, El, mode=1, n=H, out=Ys, max_ctas=mctx.gemm_ctas)
        return gu, Ys, None
    a13, b13, a2, b2 = lora
    R13, R2 = a13.shape[2], a2.shape[2]
    XA = grouped_gemm(Xs, a13.view(El * H, R13), seg_off, El, mode=1, n=R13, max_ctas=mctx.gemm_ctas)
    gu = grouped_gemm(Xs, w1.view(El * H, I_), seg_off, El, mode=1, n=2 * I_, b_alt=w3.view(El * H, I_), a2=XA,
                      b2=b13.view(El * R13, 2 * I_), max_ctas=mctx.gemm_ctas)
    hs = ACT.glu_fwd(gu[:, :I_], gu[:, I_:], act, rows_dev=used)
    HA = grouped_gemm(hs, a2.view(El * I_, R2), seg_off, El, mode=1, n=R2, max_ctas=mctx.gemm_ctas)
    Ys = grouped_gemm(hs, w2.view(El * I_, H), seg_off, El, mode=1, n=H, out=Ys, a2=HA, b2=b2.view(El * R2, H),
                      max_ctas=mctx.gemm_ctas)
    return gu, Ys, XA


def _experts_bwd_local(mctx, Xs, gu, dYs, seg_off, w1, w3, w2, act, acc, need_dw=True, lora=None, XA=None,
                       single=False):
    """Gradients of the three expert weight tensors (accumulated into ``acc`` when it already holds a chunk), of the
    low-rank factors when there are some, and the input gradient in the expert-sorted layout.  ``gu`` is overwritten
    with the pre-activation gradients.  ``single``: this call sees all the rows of the step (no token slices), so the
    weight gradients leave the GEMMs in the weights' dtype, one tensor per weight (fp32 accumulators over slices
    need a cast, and the halves of the merged gate|up accumulator a strided one: 0.18 ms per layer)."""
    I_, El, H = mctx.I, mctx.E_local, mctx.H
    nc = mctx.gemm_ctas
    used = seg_off[El:]
    hs = ACT.glu_fwd(gu[:, :I_], gu[:, I_:], act, rows_dev=used)
    if need_dw and single:
        acc["dw2_final"] = grouped_gemm(hs, dYs, seg_off, El, mode=2, m=I_, n=H, out_dtype=w2.dtype, max_ctas=nc)
    elif need_dw:
        _acc_gemm(acc, "dw2", hs, dYs, seg_off, El, I_, H, nc)
    dHA = None
    if lora is not None:
        a13, b13, a2, b2 = lora
        R13, R2 = a13.shape[2], a2.shape[2]
        HA = grouped_gemm(hs, a2.view(El * I_, R2), seg_off, El, mode=1, n=R2, max_ctas=nc)
        _acc_gemm(acc, "db2", HA, dYs, seg_off, El, R2, H, nc)
        dHA = grouped_gemm(dYs, b2.view(El * R2, H), seg_off, El, mode=1, b_mn=False, n=R2, max_ctas=nc)
        _acc_gemm(acc, "da2", hs, dHA, seg_off, El, I_, R2, nc)
    dhs = grouped_gemm(dYs, w2.view(El * I_, H), seg_off, El, mode=1, b_mn=False, n=I_, max_ctas=nc, a2=dHA,
                       b2=(a2.view(El * I_, R2) if lora is not None else None))
    ACT.glu_bwd(dhs, gu[:, :I_], gu[:, I_:], act, de=gu[:, :I_], dg=gu[:, I_:], rows_dev=used)
    if need_dw and single:
        acc["dw1_final"] = grouped_gemm(Xs, gu[:, :I_], seg_off, El, mode=2, m=H, n=I_, out_dtype=w1.dtype, max_ctas=nc)
        acc["dw3_final"] = grouped_gemm(Xs, gu[:, I_:], seg_off, El, mode=2, m=H, n=I_, out_dtype=w3.dtype, max_ctas=nc)
    elif need_dw:
        # one fp32 accumulator per weight: the cast at the end is then a contiguous one (the halves of a merged
        # [H, 2I] accumulator would need a strided cast each)
        _acc_gemm(acc, "dw1", Xs, gu[:, :I_], seg_off, El, H, I_, nc)
        _acc_gemm(acc, "dw3", Xs, gu[:, I_:], seg_off, El, H, I_, nc)
    dXs = grouped_gemm(gu[:, :I_], w1.view(El * H, I_), seg_off, El, mode=1, b_mn=False, n=H, a2=gu[:, I_:],
                       b2=w3.view(El * H, I_), max_ctas=nc)
    if lora is not None:
        _acc_gemm(acc, "db13", XA, gu, seg_off, El, R13, 2 * I_, nc)
        dXA = grouped_gemm(gu, b13.view(El * R13, 2 * I_), seg_off, El, mode=1, b_mn=False, n=R13, max_ctas=nc)
        _acc_gemm(acc, "da13", Xs, dXA, seg_off, El, H, R13, nc)
        grouped_gemm(dXA, a13.view(El * H, R13), seg_off, El, mode=1, b_mn=False, n=H, out=dXs, c=dXs, beta=1.0,
                     max_ctas=nc)
    return dXs


def _lora_grads(acc, lora, needs):
    if lora is None:
        return None, None, None, None
    keys = ("da13", "db13", "da2", "db2")
    return tuple(acc[k].to(t.dtype) if need and k in acc else None for k, t, need in zip(keys, lora, needs))


def _weight_grads(mctx, acc, w1, w3, w2, needs):
    I_ = mctx.I
    if "dw2_final" in acc:
        return (acc["dw1_final"] if needs[0] else None, acc["dw3_final"] if needs[1] else None,
                acc["dw2_final"] if needs[2] else None)
    dw1 = acc["dw1"].to(w1.dtype) if needs[0] and "dw1" in acc else None
    dw3 = acc["dw3"].to(w3.dtype) if needs[1] and "dw3" in acc else None
    dw2 = acc["dw2"].to(w2.dtype) if needs[2] and "dw2" in acc else None
    return dw1, dw3, dw2


class _Experts(torch.autograd.Function):
    """One rank owns every expert.  x [T,H], gates fp32 [T,k], idx int32 [T,k], w1/w3 [E,H,I], w2 [E,I,H] -> [T,H]."""

    @staticmethod
    def forward(ctx, x, gates, idx, w1, w3, w2, mctx: MoEContext, act: str, *lora):
        lora = lora if lora and lora[0] is not None else None
        T, H = x.shape
        dev, dt = x.device, x.dtype
        cap = mctx.cap = _round_up(T * mctx.k + mctx.E_local * 128, 128)  # exact upper bound: never overflows
        seg_off, seg_cnt, dest_row = _plan(mctx, idx, T, dev)
        Xs = torch.empty(cap, H, dtype=dt, device=dev)
        _zero_pad(mctx, Xs, seg_off, seg_cnt)
        _dispatch(mctx, x, idx, dest_row, None, _one_ptr(Xs), Xs.stride(0))
        gu, Ys, XA = _experts_fwd_local(mctx, Xs, seg_off, w1, w3, w2, act, lora=lora)
        out = _combine(mctx, _one_ptr(Ys), Ys.stride(0), idx, dest_row, gates, T, H, dt, dev)
        ctx.mctx, ctx.act, ctx.has_lora = mctx, act, lora is not None
        ctx.save_for_backward(gates, idx, w1, w3, w2, seg_off, seg_cnt, dest_row, gu, Xs, Ys, *((XA,) + lora if lora else ()))
        return out

    @staticmethod
    def backward(ctx, dout):
        mctx, act = ctx.mctx, ctx.act
        gates, idx, w1, w3, w2, seg_off, seg_cnt, dest_row, gu, Xs, Ys, *rest = ctx.saved_tensors
        XA, lora = (rest[0], tuple(rest[1:])) if ctx.has_lora else (None, None)
        dout = dout.contiguous()
        T, H = dout.shape
        El, cap = mctx.E_local, gu.shape[0]
        dev, dt = dout.device, dout.dtype
        dYs = torch.empty(cap, H, dtype=dt, device=dev)
        rgate = torch.zeros(cap, dtype=torch.float32, device=dev)
        rdots = torch.empty(cap, dtype=torch.float32, device=dev)
        _zero_pad(mctx, dYs, seg_off, seg_cnt)
        # dout rows are placed unscaled together with their routing weight; <expert output, dout> per row is the
        # routing-weight gradient, then the weight is applied in place
        rc = N.lib().fmsb_moe_dispatch_meta(dout.data_ptr(), dout.stride(0), idx.data_ptr(), dest_row.data_ptr(),
                                            gates.contiguous().data_ptr(), T * mctx.k, mctx.k, H, El, _one_ptr(dYs),
                                            dYs.stride(0), _one_ptr(rgate), 1, N.dtype_code(dt), N.stream_ptr())
        N.check(rc, "fmsb_moe_dispatch_meta")
        rc = N.lib().fmsb_moe_rowdot_scale(Ys.data_ptr(), Ys.stride(0), dYs.data_ptr(), dYs.stride(0), rgate.data_ptr(),
                                           rdots.data_ptr(), seg_off.data_ptr(), El, cap, H, N.dtype_code(dt),
                                           N.stream_ptr())
        N.check(rc, "fmsb_moe_rowdot_scale")
        acc: dict = {}
        need_dw = any(ctx.needs_input_grad[3:6])
        dXs = _experts_bwd_local(mctx, Xs, gu, dYs, seg_off, w1, w3, w2, act, acc, need_dw, lora=lora, XA=XA, single=True)
        dx = _combine(mctx, _one_ptr(dXs), dXs.stride(0), idx, dest_row, None, T, H, dt, dev)
        dgate = torch.empty(T, mctx.k, dtype=torch.float32, device=dev)
        rc = N.lib().fmsb_moe_gather_scalar(_one_ptr(rdots), idx.data_ptr(), dest_row.data_ptr(), T * mctx.k, El,
                                            dgate.data_ptr(), 1, N.stream_ptr())
        N.check(rc, "fmsb_moe_gather_scalar")
        dw1, dw3, dw2 = _weight_grads(mctx, acc, w1, w3, w2, ctx.needs_input_grad[3:6])
        return (dx, dgate, None, dw1, dw3, dw2, None, None) + (_lora_grads(acc, lora, ctx.needs_input_grad[8:12]) if lora else ())


# ------------------------------------------------------------------------------------------------ expert parallel
class _Chunk:
    """Plan and buffers of one token slice of an expert-parallel call."""
    __slots__ = ("t0", "t1", "s", "seg_off", "seg_cnt", "dest_row", "hit", "stage_row", "stage_cnt", "Xs", "gu", "Ys",
                 "dYs", "rgate", "dXs", "XA")


def _stage_plan(sh: _EPShared, idx_c, dest_row, n, dev):
    hit = torch.empty(max(n, 1), sh.world, dtype=torch.int32, device=dev)
    stage_row = torch.empty(max(n, 1), sh.world, dtype=torch.int32, device=dev)
    stage_cnt = torch.empty(sh.world, dtype=torch.int32, device=dev)
    scratch = torch.empty(max(1, -(-n * sh.world // 1024)) * sh.world, dtype=torch.int32, device=dev)
    rc = N.lib().fmsb_moe_stage_plan(N.ptr(idx_c) if n else None, N.ptr(dest_row) if n else None, n, sh.k, sh.E_local,
                                     sh.world, sh.stage_base.data_ptr(), hit.data_ptr(), stage_row.data_ptr(),
                                     stage_cnt.data_ptr(), scratch.data_ptr(), N.stream_ptr())
    N.check(rc, "fmsb_moe_stage_plan")
    return hit, stage_row, stage_cnt


def _push(sh: _EPShared, ch: _Chunk, rows, idx, gates, chan):
    """Communication stream: store the slice's rows once per destination rank, then the barrier after which every
    rank's staging block is complete."""
    n = ch.t1 - ch.t0
    x = rows[ch.t0:ch.t1]
    g = gates[ch.t0:ch.t1] if gates is not None else None
    rc = N.lib().fmsb_moe_dispatch_staged(
        x.data_ptr() if n else None, rows.stride(0), idx[ch.t0:ch.t1].data_ptr() if n else None,
        ch.dest_row.data_ptr() if n else None, N.ptr(g) if n else None, ch.stage_row.data_ptr(), ch.stage_cnt.data_ptr(), n,
        sh.k, sh.H, sh.E_local, sh.world, sh.rank, sh.ptrs[("x", ch.s)], sh.H, sh.ptrs[("slot", ch.s)],
        sh.ptrs[("gate", ch.s)], sh.ptrs[("cnt", ch.s)], N.dtype_code(rows.dtype), N.stream_ptr())
    N.check(rc, "fmsb_moe_dispatch_staged")
    sh.comm.barrier(chan)


def _replicate(sh: _EPShared, ch: _Chunk, buf, slot_out=None):
    n_rows = sh.world * sh.Tbc
    rc = N.lib().fmsb_moe_replicate(sh.local_ptr("x", ch.s), sh.H, sh.local_ptr("slot", ch.s),
                                    sh.local_ptr("gate", ch.s) if slot_out is not None else None, N.ptr(slot_out), n_rows,
                                    sh.Tbc, sh.local_ptr("cnt", ch.s), sh.k, sh.H, buf.data_ptr(), buf.stride(0),
                                    N.dtype_code(buf.dtype), N.stream_ptr())
    N.check(rc, "fmsb_moe_replicate")


def _prereduce(sh: _EPShared, ch: _Chunk, buf, weighted: bool):
    n_rows = sh.world * sh.Tbc
    rc = N.lib().fmsb_moe_prereduce(buf.data_ptr(), buf.stride(0), sh.local_ptr("slot", ch.s),
                                    sh.local_ptr("gate", ch.s) if weighted else None, n_rows, sh.Tbc,
                                    sh.local_ptr("cnt", ch.s), sh.k, sh.H, sh.local_ptr("y", ch.s), sh.H,
                                    N.dtype_code(buf.dtype), N.stream_ptr())
    N.check(rc, "fmsb_moe_prereduce")


def _pull(sh: _EPShared, mctx, ch: _Chunk, out, chan):
    """Communication stream: barrier (every owner's reduced rows are written), then one row per (token, rank) is
    read back and summed."""
    sh.comm.barrier(chan)
    n = ch.t1 - ch.t0
    if n:
        _combine(mctx, sh.ptrs[("y", ch.s)], sh.H, ch.hit, ch.stage_row, None, n, sh.H, out.dtype, out.device,
                 out=out[ch.t0:ch.t1], k=sh.world, e_local=1, world=sh.world)


def _pipeline(sh: _EPShared, chunks, push, compute, pull):
    """push(c), pull(c) on the communication stream, compute(c) on the caller's stream; slice c+1 is pushed while
    slice c computes, slice c is pulled while slice c+1 computes.  Staging set c % 2 is reused by slice c+2 only
    after pull(c) (whose barrier every rank passes after its compute(c))."""
    main = torch.cuda.current_stream(sh.device)
    comm = sh.stream
    C = len(chunks)
    ready = [torch.cuda.Event() for _ in range(C)]
    done = [torch.cuda.Event() for _ in range(C)]

    def do_push(c):
        with torch.cuda.stream(comm):
            push(chunks[c])
            ready[c].record(comm)

    start = torch.cuda.Event()
    start.record(main)
    comm.wait_event(start)
    do_push(0)
    if C > 1:
        do_push(1)
    for c in range(C):
        main.wait_event(ready[c])
        compute(chunks[c])
        done[c].record(main)
        with torch.cuda.stream(comm):
            comm.wait_event(done[c])
            pull(chunks[c])
        if c + 2 < C:
            do_push(c + 2)
    end = torch.cuda.Event()
    end.record(comm)
    main.wait_event(end)


class _ExpertsEP(torch.autograd.Function):
    """Expert-parallel form: this rank owns ``E / world`` experts (w1/w3 [E_local,H,I], w2 [E_local,I,H])."""

    @staticmethod
    def forward(ctx, x, gates, idx, w1, w3, w2, mctx: MoEContext, act: str, *lora):
        lora = lora if lora and lora[0] is not None else None
        T, H = x.shape
        dev, dt = x.device, x.dtype
        sh = mctx.ensure_shared(T, dt, dev)
        gates = gates.contiguous()
        Tc = max(1, -(-T // sh.C))
        chunks = []
        for c in range(sh.C):
            ch = _Chunk()
            ch.t0, ch.t1, ch.s = min(T, c * Tc), min(T, (c + 1) * Tc), c % 2
            n = ch.t1 - ch.t0
            ch.seg_off, ch.seg_cnt, ch.dest_row = _plan(mctx, idx[ch.t0:ch.t1], n, dev, cap=sh.cap)
            ch.hit, ch.stage_row, ch.stage_cnt = _stage_plan(sh, idx[ch.t0:ch.t1], ch.dest_row, n, dev)
            chunks.append(ch)
        out = torch.empty(T, H, dtype=dt, device=dev)
        for ch in chunks:
            ch.Xs = torch.empty(sh.cap, H, dtype=dt, device=dev)

        # The data-movement kernels of a slice (store to the owners, replicate into the expert-sorted buffer; reduce per
        # staged row, read back) run on the communication stream, so that they overlap the grouped GEMMs of the
        # neighbouring slice, which are all the compute stream does.
        def push(ch):
            _push(sh, ch, x, idx, gates, BAR_A)
            _zero_pad(mctx, ch.Xs, ch.seg_off, ch.seg_cnt)
            _replicate(sh, ch, ch.Xs)

        def compute(ch):
            ch.gu, ch.Ys, ch.XA = _experts_fwd_local(mctx, ch.Xs, ch.seg_off, w1, w3, w2, act, lora=lora)

        def pull(ch):
            _prereduce(sh, ch, ch.Ys, weighted=True)
            _pull(sh, mctx, ch, out, BAR_B)

        _pipeline(sh, chunks, push, compute, pull)
        ctx.mctx, ctx.act, ctx.chunks, ctx.has_lora = mctx, act, chunks, lora is not None
        ctx.save_for_backward(gates, idx, w1, w3, w2, *(lora or ()))
        return out

    @staticmethod
    def backward(ctx, dout):
        mctx, act, chunks = ctx.mctx, ctx.act, ctx.chunks
        gates, idx, w1, w3, w2, *rest = ctx.saved_tensors
        lora = tuple(rest) if ctx.has_lora else None
        sh = mctx.shared
        dout = dout.contiguous()
        T, H = dout.shape
        dev, dt = dout.device, dout.dtype
        El = mctx.E_local
        dx = torch.empty(T, H, dtype=dt, device=dev)
        dgate = torch.zeros(T, mctx.k, dtype=torch.float32, device=dev)
        acc: dict = {}
        need_dw = any(ctx.needs_input_grad[3:6])

        for ch in chunks:
            ch.dYs = torch.empty(sh.cap, H, dtype=dt, device=dev)
            ch.rgate = torch.zeros(sh.cap, dtype=torch.float32, device=dev)

        def push(ch):
            _push(sh, ch, dout, idx, gates, BAR_C)
            _zero_pad(mctx, ch.dYs, ch.seg_off, ch.seg_cnt)
            # unscaled dout rows and the routing weight of every received row; the owner forms <expert output, dout>
            # per row (read back by the source, 4 bytes per pair) and applies the weight in place
            _replicate(sh, ch, ch.dYs, slot_out=ch.rgate)
            rc = N.lib().fmsb_moe_rowdot_scale(ch.Ys.data_ptr(), ch.Ys.stride(0), ch.dYs.data_ptr(), ch.dYs.stride(0),
                                               ch.rgate.data_ptr(), sh.local_ptr("rdots", ch.s), ch.seg_off.data_ptr(),
                                               El, sh.cap, H, N.dtype_code(dt), N.stream_ptr())
            N.check(rc, "fmsb_moe_rowdot_scale")

        def compute(ch):
            ch.dXs = _experts_bwd_local(mctx, ch.Xs, ch.gu, ch.dYs, ch.seg_off, w1, w3, w2, act, acc, need_dw, lora=lora,
                                        XA=ch.XA, single=len(chunks) == 1)

        def pull(ch):
            _prereduce(sh, ch, ch.dXs, weighted=False)
            _pull(sh, mctx, ch, dx, BAR_D)
            n = ch.t1 - ch.t0
            if n:
                rc = N.lib().fmsb_moe_gather_scalar(sh.ptrs[("rdots", ch.s)], idx[ch.t0:ch.t1].data_ptr(),
                                                    ch.dest_row.data_ptr(), n * mctx.k, El,
                                                    dgate[ch.t0:ch.t1].data_ptr(), sh.world, N.stream_ptr())
                N.check(rc, "fmsb_moe_gather_scalar")

        _pipeline(sh, chunks, push, compute, pull)
        for ch in chunks:  # only now: the communication stream has finished reading them
            ch.Xs = ch.gu = ch.Ys = ch.dYs = ch.rgate = ch.dXs = ch.XA = None
        dw1, dw3, dw2 = _weight_grads(mctx, acc, w1, w3, w2, ctx.needs_input_grad[3:6])
        return (dx, dgate, None, dw1, dw3, dw2, None, None) + (_lora_grads(acc, lora, ctx.needs_input_grad[8:12]) if lora else ())


def pack_expert_lora(a1, b1, a3, b3, a2, b2):
    """Low-rank factors of the three expert projections in the layout the grouped kernel reads.

    Inputs per projection: ``A [El, in, r]`` and ``B [El, r, out]``.  Returns ``(A13 [El, H, R13], B13 [El, R13, 2I],
    A2 [El, I, R2], B2 [El, R2, H])`` with gate and up side by side (``A13 = [A1 | A3 | 0]``, ``B13`` block-diagonal)
    and the ranks padded with zeros to the kernel's 64-element contraction block, so that one group's block never
    reaches into the next group's rows.  Plain tensor ops: autograd carries the gradients back to the six factors."""
    r = a1.shape[2]
    I_ = b1.shape[2]
    R13, R2 = _round_up(2 * r, 64), _round_up(r, 64)
    z = a1.new_zeros
    El, H = a1.shape[0], a1.shape[1]
    A13 = torch.cat([a1, a3, z(El, H, R13 - 2 * r)], dim=2)
    B13 = torch.cat([torch.cat([b1, z(El, r, I_)], dim=2), torch.cat([z(El, r, I_), b3], dim=2),
                     z(El, R13 - 2 * r, 2 * I_)], dim=1)
    A2 = torch.cat([a2, z(El, I_, R2 - r)], dim=2)
    B2 = torch.cat([b2, z(El, R2 - r, b2.shape[2])], dim=1)
    return A13.contiguous(), B13.contiguous(), A2.contiguous(), B2.contiguous()


def experts_forward(x, gates, idx, w1, w3, w2, mctx: MoEContext, act="silu", lora=None):
    """``lora``: the four tensors of :func:`pack_expert_lora`, or None."""
    fn = _ExpertsEP if mctx.world > 1 else _Experts
    return fn.apply(x, gates, idx, w1, w3, w2, mctx, act, *(lora or ()))
