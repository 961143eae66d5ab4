"""Context parallelism for Mamba2: one sequence is split into contiguous slices over the ranks of a group.

The SSD recurrence is linear in the state, so the state that ENTERS rank ``r``'s slice is
``H_in(r) = sum_{j<r} (prod_{j<i<r} P_i) F_j``, where ``F_j`` is rank ``j``'s zero-start final state and
``P_j = exp(sum of dt*A over slice j)`` its total decay.  Inside the scan, once the chunk states of the slice are known,
the kernel of the zero-start inter-chunk recurrence stores ``(F, log P)`` straight into a slot of every LATER rank's
symmetric buffer (peer stores from the threads that computed them, release flag by the last CTA: ``csrc/cp.cu``); a
second kernel waits (bounded) for the earlier ranks' flags and combines the prefix on the device; the recurrence
proper then starts from ``H_in``, so the outputs need no correction pass.  This is the "allgather" flavour the
reference defaults to (fms_acceleration_mcp/framework_plugin_mcp.py:29-44).  The backward mirrors it right to left:
``dH_in`` becomes ``dF_j`` / ``dlog P_j`` for the earlier ranks (one kernel, pushed), and what the later ranks send runs
back through the zero-start recurrence.  The conv1d halo (last ``d_conv - 1`` rows of the previous slice) and the
label that the last position predicts go to the neighbour only.

``backend="library"`` (or ``FMSB_CP_BACKEND=library``; the default on a CPU) states the same exchange with the process
group's collectives, NCCL on GPUs and gloo on CPUs: every rank scans its slice from a zero state, the
``(F, log P)`` pairs are all-gathered, the prefix is combined locally and the entering state's contribution is added
to the outputs; the halo is an all-gather of every rank's last rows.  It is the like-for-like library form of the
fused path (what the reference's external ``Mamba2CP`` module does with ``torch.distributed``) and the form that CPU
tests run.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch
import torch.distributed as dist

from .. import _native as NV
from ..ops import mamba as MB

P_, I_, L_, U_ = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_uint
NV.declare("fmsb_cp_push", [P_, L_, P_, P_, L_, I_, I_, I_, I_, U_, I_, P_, P_])
NV.declare("fmsb_cp_wait", [P_, I_, I_, I_, I_, I_, U_, P_, P_])
NV.declare("fmsb_cp_state_push", [P_, P_, P_, I_, I_, I_, P_, L_, P_, I_, I_, U_, P_, I_, P_])
NV.declare("fmsb_cp_prefix_fwd", [P_, L_, P_, I_, U_, I_, I_, P_, P_, P_])
NV.declare("fmsb_cp_prefix_bwd", [P_, P_, L_, P_, P_, I_, I_, U_, I_, I_, P_, P_])
NV.declare("fmsb_cp_sum_bwd", [P_, L_, P_, I_, I_, U_, I_, I_, P_, P_, P_, P_])

CH_STATE_F, CH_STATE_B, CH_HALO_F, CH_HALO_B = 20, 21, 22, 23


class _Slots:
    """Symmetric slot buffer: ``world`` slots of ``slot_bytes`` per rank (slot j = data sent by rank j)."""

    def __init__(self, comm, slot_bytes: int, device):
        from .symm import SymmBuffer

        self.slot_bytes = (slot_bytes + 255) // 256 * 256
        self.buf = SymmBuffer(self.slot_bytes * comm.world, comm.group, device)


class ContextParallel:
    """Communication state shared by all Mamba2 layers of a model (buffers are reused layer after layer)."""

    def __init__(self, group: Optional[dist.ProcessGroup] = None, device=None, impl: str = "allgather",
                 recompute: bool = False, backend: Optional[str] = None):
        from .symm import Communicator

        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        # impl: "allgather" and "serial" give the same entering state.  Both use the all-to-later push: through
        # NVSwitch every later rank is one hop away at full bandwidth and a (state, decay) pair is a few MB, so a
        # rank-to-rank chain would only add world-1 latencies to the last rank.  recompute: the scan keeps only its
        # inputs and rebuilds the per-chunk entering states in the backward.
        self.impl, self.recompute = impl, recompute
        self.backend = backend or os.environ.get("FMSB_CP_BACKEND") or ("fused" if self.device.type == "cuda" else "library")
        if self.backend not in ("fused", "library"):
            raise ValueError(f"unknown context-parallel backend {self.backend!r}")
        self._slots = {}
        self._hooks = {}
        if self.backend == "library":
            self.comm = None  # no peer memory: the process group's collectives carry everything
            return
        self.comm = Communicator(self.group, self.device)
        self._counter = torch.zeros(4, dtype=torch.int32, device=self.device)  # "last CTA" counters of the fused kernels

    # ------------------------------------------------------------------ primitive: push to later / earlier ranks
    def _exchange(self, payload: torch.Tensor, chan: int, direction: int, tag=None, span: int = 0) -> torch.Tensor:
        """Send ``payload`` (contiguous) to the ``span`` ranks after (direction=+1) or before (-1) this one (0: all of
        them); returns the received slots as ``[world, numel]`` (only the slots of the sending side are meaningful)."""
        nbytes = payload.numel() * payload.element_size()
        # one slot set per (channel, layer): an earlier rank may run several layers ahead of a later one, so a
        # slot is never reused before the step's backward (which needs the later ranks) has drained it
        key = (chan, nbytes, payload.dtype, tag)
        if key not in self._slots:
            self._slots[key] = _Slots(self.comm, nbytes, self.device)
        slots = self._slots[key]
        epoch = self.comm.next_epoch(chan)
        st = NV.status_word(self.device)
        sig = self.comm.signals.ptr_array(chan * self.world * 4)
        rc = NV.lib().fmsb_cp_push(payload.data_ptr(), nbytes, slots.buf.ptr_array(), sig, slots.slot_bytes, self.rank,
                                   self.world, direction, 0, epoch, span, st.data_ptr(), NV.stream_ptr())
        NV.check(rc, "fmsb_cp_push")
        rc = NV.lib().fmsb_cp_wait(self.comm.signals.ptrs[self.rank] + chan * self.world * 4, self.rank, self.world,
                                   direction, span, 0, epoch, st.data_ptr(), NV.stream_ptr())
        NV.check(rc, "fmsb_cp_wait")
        numel = payload.numel()
        view = slots.buf.local.view(self.world, slots.slot_bytes)[:, :nbytes].view(payload.dtype).view(self.world, numel)
        return view

    # ------------------------------------------------------------------ conv halo
    def exchange_halo(self, xBC: torch.Tensor, k: int, layer=None) -> torch.Tensor:
        if self.backend == "library":
            # every rank's last k rows, gathered; mine are the previous rank's (zeros on rank 0).  The zero-weight
            # term keeps the gather in every rank's graph, so that its backward (a collective) runs everywhere.
            tails = _GatherTokens.apply(xBC[-k:].contiguous(), self.group)
            halo = tails[(self.rank - 1) * k:self.rank * k] if self.rank > 0 else torch.zeros_like(xBC[-k:])
            return halo + 0.0 * tails.sum()
        return _HaloExchange.apply(xBC, self, k, layer)

    # ------------------------------------------------------------------ scan
    def scan(self, x, dt, A, B, C, D, Q, layer=None):
        """Context-parallel SSD scan of this rank's slice; returns y."""
        if self.backend == "library":
            return self._scan_library(x, dt, A, B, C, D, Q)
        hook = self._hooks.get(layer)
        if hook is None:
            hook = self._hooks[layer] = StateHandoff(self, layer)
        y, _ = MB.ssd_scan(x, dt, A, B, C, D, None, Q, recompute=self.recompute, cp=hook)
        return y

    def _scan_library(self, x, dt, A, B, C, D, Q):
        """Zero-start scan of the slice, all-gather of every rank's ``(final state, log total decay)``, prefix combine
        on this rank, then the entering state's contribution ``exp(cumsum dt A) (C . H_in)`` added to the outputs.
        Every piece is differentiable (the gather's backward is the matching reduce-scatter), so the state gradients
        travel right to left through the same collectives."""
        nh, P = x.shape[1], x.shape[2]
        N = B.shape[2]
        y0, F = MB.ssd_scan(x, dt, A, B, C, D, None, Q, recompute=self.recompute)
        logP = (dt.float() * A.float()[None, :]).sum(0)
        mine = torch.cat([F.float().reshape(nh, P * N), logP[:, None]], dim=1)[None]     # [1, nh, P*N + 1]
        every = _GatherTokens.apply(mine, self.group)                                    # [world, nh, P*N + 1]
        Fs, lPs = every[..., :-1].reshape(self.world, nh, P, N), every[..., -1]
        h_in = prefix_state(Fs, lPs, self.rank) + 0.0 * every.sum()  # rank 0 too keeps the gather in its graph
        return MB.state_correction(y0, h_in, dt, A, C, Q)

    # ------------------------------------------------------------------ loss helpers
    def shift_labels(self, flat_labels: torch.Tensor) -> torch.Tensor:
        """Next-token targets for this slice: the last position takes the first label of the NEXT rank's slice."""
        first = flat_labels[:1].contiguous()
        if self.backend == "library":
            firsts = [torch.empty_like(first) for _ in range(self.world)]
            dist.all_gather(firsts, first, group=self.group)
            nxt = firsts[self.rank + 1] if self.rank + 1 < self.world else torch.full_like(first, -100)
            return torch.cat([flat_labels[1:], nxt])
        recv = self._exchange(first, CH_HALO_B, -1, span=1)                   # from the next rank, slot = sender
        nxt = recv[self.rank + 1] if self.rank + 1 < self.world else torch.full_like(first, -100)
        return torch.cat([flat_labels[1:], nxt.to(flat_labels.dtype)])

    def global_count(self, mask: torch.Tensor) -> torch.Tensor:
        n = mask.sum().float().reshape(1)
        dist.all_reduce(n, group=self.group)
        return n.clamp(min=1)


def prefix_state(Fs: torch.Tensor, lPs: torch.Tensor, r: int) -> torch.Tensor:
    """PyTorch statement of the device-side prefix combine (``cp_prefix_fwd_kernel``): state entering rank ``r``'s slice from the zero-initial-state final states ``Fs [>=r, nh, P, N]`` and the log
    total decays ``lPs [>=r, nh]`` of the earlier ranks: left to right, ``H <- exp(lP_j) H + F_j``."""
    h = torch.zeros_like(Fs[0], dtype=torch.float32)
    for j in range(r):
        h = torch.exp(lPs[j])[:, None, None] * h + Fs[j]
    return h


def prefix_state_grads(dh: torch.Tensor, Fs: torch.Tensor, lPs: torch.Tensor, r: int, world: int):
    """PyTorch statement of ``cp_prefix_bwd_push_kernel``: gradients of :func:`prefix_state` with respect to every earlier rank's ``F_j`` and ``lP_j``:
    ``(dF [world, nh, P, N], dlP [world, nh])``, rows ``>= r`` zero."""
    nh = dh.shape[0]
    dF = torch.zeros(world, *dh.shape, dtype=torch.float32, device=dh.device)
    dlP = torch.zeros(world, nh, dtype=torch.float32, device=dh.device)
    g = dh.float().clone()
    # prefixes H^{(j)}: the state after absorbing the ranks below j
    prefix = [torch.zeros_like(g)]
    for j in range(r):
        prefix.append(torch.exp(lPs[j])[:, None, None] * prefix[-1] + Fs[j])
    for j in range(r - 1, -1, -1):
        dF[j] = g
        dlP[j] = (g * prefix[j]).sum((1, 2)) * torch.exp(lPs[j])
        g = torch.exp(lPs[j])[:, None, None] * g
    return dF, dlP


class StateHandoff:
    """The hook the chunked scan calls (``ops/mamba.py``): ``forward`` hands this slice's zero-start final state to the
    later ranks from inside the state kernel and returns the state entering the slice; ``backward`` turns the gradient
    of the entering state into the earlier ranks' shares and returns what the later ranks sent for this slice.  One
    set of slots per layer: an early rank may run several layers ahead of a late one."""

    def __init__(self, cp: ContextParallel, layer):
        self.cp, self.layer = cp, layer
        self.fwd = self.bwd = None
        self.slot_elems = 0

    def _ensure(self, nh: int, PN: int):
        from .symm import SymmBuffer

        if self.fwd is None:
            cp = self.cp
            self.slot_elems = (nh * PN + nh + 63) // 64 * 64
            nbytes = cp.world * self.slot_elems * 4
            self.fwd = SymmBuffer(nbytes, cp.group, cp.device)
            self.bwd = SymmBuffer(nbytes, cp.group, cp.device)

    def forward(self, S, Ltot, hprev0, nc, nh, PN, dtp):
        cp = self.cp
        self._ensure(nh, PN)
        st = NV.status_word(cp.device)
        epoch = cp.comm.next_epoch(CH_STATE_F)
        sig_off = CH_STATE_F * cp.world * 4
        rc = NV.lib().fmsb_cp_state_push(S.data_ptr(), Ltot.data_ptr(), hprev0.data_ptr(), nc, nh, PN,
                                         self.fwd.ptr_array(), self.slot_elems, cp.comm.signals.ptr_array(sig_off),
                                         cp.rank, cp.world, epoch, cp._counter.data_ptr(), NV.dtype_code(dtp),
                                         NV.stream_ptr())
        NV.check(rc, "fmsb_cp_state_push")
        h_in = torch.empty(nh, PN, dtype=torch.float32, device=cp.device)
        rc = NV.lib().fmsb_cp_prefix_fwd(self.fwd.local.data_ptr(), self.slot_elems,
                                         cp.comm.signals.ptrs[cp.rank] + sig_off, cp.rank, epoch, nh, PN,
                                         h_in.data_ptr(), st.data_ptr(), NV.stream_ptr())
        NV.check(rc, "fmsb_cp_prefix_fwd")
        return h_in

    def backward(self, dh_in, nh: int, PN: int):
        cp = self.cp
        st = NV.status_word(cp.device)
        epoch = cp.comm.next_epoch(CH_STATE_B)
        sig_off = CH_STATE_B * cp.world * 4
        dh = dh_in.float().contiguous()
        rc = NV.lib().fmsb_cp_prefix_bwd(dh.data_ptr(), self.fwd.local.data_ptr(), self.slot_elems, self.bwd.ptr_array(),
                                         cp.comm.signals.ptr_array(sig_off), cp.rank, cp.world, epoch, nh, PN,
                                         cp._counter[1:].data_ptr(), NV.stream_ptr())
        NV.check(rc, "fmsb_cp_prefix_bwd")
        dF = torch.empty(nh, PN, dtype=torch.float32, device=cp.device)
        dlogP = torch.empty(nh, dtype=torch.float32, device=cp.device)
        rc = NV.lib().fmsb_cp_sum_bwd(self.bwd.local.data_ptr(), self.slot_elems,
                                      cp.comm.signals.ptrs[cp.rank] + sig_off, cp.rank, cp.world, epoch, nh, PN,
                                      dF.data_ptr(), dlogP.data_ptr(), st.data_ptr(), NV.stream_ptr())
        NV.check(rc, "fmsb_cp_sum_bwd")
        return dF, dlogP


def _exchange_rows(cp: ContextParallel, payload: torch.Tensor, chan: int, direction: int, tag=None,
                   span: int = 0) -> torch.Tensor:
    """Row ``j`` of ``payload`` is delivered to rank ``j`` (only ranks on the ``direction`` side are served); returns
    ``[world (sender), row]``."""
    world, row = payload.shape
    nbytes = row * payload.element_size()
    key = (chan, nbytes, payload.dtype, "rows", tag)
    if key not in cp._slots:
        cp._slots[key] = _Slots(cp.comm, nbytes, cp.device)
    slots = cp._slots[key]
    epoch = cp.comm.next_epoch(chan)
    st = NV.status_word(cp.device)
    sig = cp.comm.signals.ptr_array(chan * cp.world * 4)
    rc = NV.lib().fmsb_cp_push(payload.data_ptr(), nbytes, slots.buf.ptr_array(), sig, slots.slot_bytes, cp.rank, cp.world,
                               direction, 1, epoch, span, st.data_ptr(), NV.stream_ptr())
    NV.check(rc, "fmsb_cp_push")
    rc = NV.lib().fmsb_cp_wait(cp.comm.signals.ptrs[cp.rank] + chan * cp.world * 4, cp.rank, cp.world, direction, span,
                               0, epoch, st.data_ptr(), NV.stream_ptr())
    NV.check(rc, "fmsb_cp_wait")
    return slots.buf.local.view(cp.world, slots.slot_bytes)[:, :nbytes].view(payload.dtype).view(cp.world, row)


class _HaloExchange(torch.autograd.Function):
    """Last ``k`` rows of the previous rank's conv input (zeros on rank 0)."""

    @staticmethod
    def forward(ctx, xBC, cp: ContextParallel, k: int, layer):
        tail = xBC[-k:].contiguous()
        recv = cp._exchange(tail.reshape(-1), CH_HALO_F, +1, layer, span=1)
        ctx.cp, ctx.k, ctx.shape, ctx.layer = cp, k, xBC.shape, layer
        if cp.rank == 0:
            return torch.zeros_like(tail)
        return recv[cp.rank - 1].view_as(tail).clone()

    @staticmethod
    def backward(ctx, dhalo):
        cp, k = ctx.cp, ctx.k
        # the gradient of my halo belongs to the previous rank's last k rows
        payload = torch.zeros(cp.world, dhalo.numel(), dtype=dhalo.dtype, device=dhalo.device)
        if cp.rank > 0:
            payload[cp.rank - 1] = dhalo.reshape(-1)
        recv = _exchange_rows(cp, payload.contiguous(), CH_HALO_B + 4, -1, ctx.layer, span=1)
        dx = torch.zeros(ctx.shape, dtype=dhalo.dtype, device=dhalo.device)
        if cp.rank + 1 < cp.world:
            dx[-k:] = recv[cp.rank + 1].view(k, -1)
        return dx, None, None, None


# ------------------------------------------------------------------------------------------------
# Attention layers of hybrid models under context parallelism (library collectives)
# ------------------------------------------------------------------------------------------------
class _GatherTokens(torch.autograd.Function):
    """All-gather along the token axis over the context-parallel group; the backward sums every rank's gradient of
    the gathered tensor and keeps this rank's slice (a reduce-scatter, stated with all_reduce so that gloo runs it)."""

    @staticmethod
    def forward(ctx, t, group):
        ctx.group, ctx.n = group, t.shape[0]
        world = dist.get_world_size(group)
        parts = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(parts, t.contiguous(), group=group)
        return torch.cat(parts, dim=0)

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        dist.all_reduce(g, group=ctx.group)
        r = dist.get_rank(ctx.group)
        return g[r * ctx.n:(r + 1) * ctx.n], None


def cp_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, group, scaling: float,
                 q_block: int = 1024) -> torch.Tensor:
    """Causal attention of ONE sequence whose tokens are split evenly and in order over the ranks of ``group``.

    ``q [Tl, nh, d]``, ``k`` / ``v [Tl, nkv, d]`` are this rank's slice (rank r holds tokens ``[r Tl, (r + 1) Tl)``).
    Keys and values of all ranks are gathered, query ``i`` of this rank attends the keys ``0 .. r Tl + i``.  Queries
    are processed in blocks of ``q_block`` rows so that the explicit mask stays small.  Differentiable (the gradient
    of the gathered keys / values is summed over the ranks).  Library form: the hybrid models' few attention layers
    under the Mamba context-parallel plugin, where the reference relies on torch's experimental context-parallel
    attention (fms_acceleration_mcp/utils/utils.py:64-80)."""
    import torch.nn.functional as F

    r = dist.get_rank(group)
    Tl, nh, d = q.shape
    nkv = k.shape[1]
    K = _GatherTokens.apply(k, group)[: (r + 1) * Tl]
    V = _GatherTokens.apply(v, group)[: (r + 1) * Tl]
    rep = nh // nkv
    Kh = K.repeat_interleave(rep, dim=1).transpose(0, 1).unsqueeze(0)  # [1, nh, Tk, d]
    Vh = V.repeat_interleave(rep, dim=1).transpose(0, 1).unsqueeze(0)
    outs = []
    kpos = torch.arange((r + 1) * Tl, device=q.device)
    for s in range(0, Tl, q_block):
        e = min(Tl, s + q_block)
        last = r * Tl + e  # keys beyond the block's last query are masked for every row of the block: cut them off
        qh = q[s:e].transpose(0, 1).unsqueeze(0)
        mask = kpos[None, :last] <= (r * Tl + torch.arange(s, e, device=q.device))[:, None]
        o = F.scaled_dot_product_attention(qh, Kh[:, :, :last], Vh[:, :, :last], attn_mask=mask, scale=scaling)
        outs.append(o.squeeze(0).transpose(0, 1))
    return torch.cat(outs, dim=0)
