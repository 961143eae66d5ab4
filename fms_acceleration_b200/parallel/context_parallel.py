"""Context parallelism for Mamba2: one sequence is split into contiguous slices over the ranks of a group.

The SSD recurrence is linear in the state, so rank ``r`` can scan its slice with a zero initial state and only needs
the state that ENTERS its slice, ``H_in(r) = sum_{j<r} (prod_{j<i<r} P_i) F_j``, where ``F_j`` is rank ``j``'s
zero-initial-state final state and ``P_j = exp(sum of dt*A over slice j)`` its total decay.  Every rank writes its
``(F, P)`` pair straight into a slot of every LATER rank's symmetric buffer (peer stores, ``csrc/cp.cu``) and
release-flags it; the receivers combine the prefix locally and run the inter-chunk pass with ``h0 = H_in``.
This is the "allgather" flavour the reference defaults to (fms_acceleration_mcp/framework_plugin_mcp.py:29-44); the
backward pass mirrors it right-to-left with the gradient of the entering state.  The conv1d halo (last
``d_conv - 1`` rows of the previous slice) travels the same way.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.distributed as dist

from .. import _native as NV
from ..ops import mamba as MB

P_, I_, L_, U_ = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_uint
NV.declare("fmsb_cp_push", [P_, L_, P_, P_, L_, I_, I_, I_, I_, U_, P_, P_])
NV.declare("fmsb_cp_wait", [P_, I_, I_, I_, I_, I_, U_, P_, P_])

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
                 recompute: bool = False):
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
        self.comm = Communicator(self.group, self.device)
        self._slots = {}

    # ------------------------------------------------------------------ primitive: push to later / earlier ranks
    def _exchange(self, payload: torch.Tensor, chan: int, direction: int, tag=None) -> torch.Tensor:
        """Send ``payload`` (contiguous) to every rank after (direction=+1) or before (-1) this one; returns the
        received slots as ``[world, numel]`` (only the slots of the sending side are meaningful)."""
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
                                   self.world, direction, 0, epoch, st.data_ptr(), NV.stream_ptr())
        NV.check(rc, "fmsb_cp_push")
        rc = NV.lib().fmsb_cp_wait(self.comm.signals.ptrs[self.rank] + chan * self.world * 4, self.rank, self.world,
                                   direction, 0, 0, epoch, st.data_ptr(), NV.stream_ptr())
        NV.check(rc, "fmsb_cp_wait")
        numel = payload.numel()
        view = slots.buf.local.view(self.world, slots.slot_bytes)[:, :nbytes].view(payload.dtype).view(self.world, numel)
        return view

    # ------------------------------------------------------------------ conv halo
    def exchange_halo(self, xBC: torch.Tensor, k: int, layer=None) -> torch.Tensor:
        return _HaloExchange.apply(xBC, self, k, layer)

    # ------------------------------------------------------------------ scan
    def scan(self, x, dt, A, B, C, D, Q, layer=None):
        """Context-parallel SSD scan of this rank's slice; returns y."""
        nh = x.shape[1]
        # pass 1: zero-initial-state scan gives the slice's final state F and total decay P
        y0, F_local = MB.ssd_scan(x, dt, A, B, C, D, None, Q, recompute=self.recompute)
        logP = (dt.float() * A.float()[None, :]).sum(0)                       # [nh]
        h_in = _StateExchange.apply(F_local, logP, self, layer)
        # the entering state only adds  exp(L_global(t)) * C_t . H_in  to every output row of the slice
        return MB.state_correction(y0, h_in, dt, A, C, Q)

    # ------------------------------------------------------------------ loss helpers
    def shift_labels(self, flat_labels: torch.Tensor) -> torch.Tensor:
        """Next-token targets for this slice: the last position takes the first label of the NEXT rank's slice."""
        first = flat_labels[:1].contiguous()
        recv = self._exchange(first, CH_HALO_B, -1)                           # from later ranks, slot = sender
        nxt = recv[self.rank + 1] if self.rank + 1 < self.world else torch.full_like(first, -100)
        return torch.cat([flat_labels[1:], nxt.to(flat_labels.dtype)])

    def global_count(self, mask: torch.Tensor) -> torch.Tensor:
        n = mask.sum().float().reshape(1)
        dist.all_reduce(n, group=self.group)
        return n.clamp(min=1)


def prefix_state(Fs: torch.Tensor, lPs: torch.Tensor, r: int) -> torch.Tensor:
    """State entering rank ``r``'s slice from the zero-initial-state final states ``Fs [>=r, nh, P, N]`` and the log
    total decays ``lPs [>=r, nh]`` of the earlier ranks: left to right, ``H <- exp(lP_j) H + F_j``."""
    h = torch.zeros_like(Fs[0], dtype=torch.float32)
    for j in range(r):
        h = torch.exp(lPs[j])[:, None, None] * h + Fs[j]
    return h


def prefix_state_grads(dh: torch.Tensor, Fs: torch.Tensor, lPs: torch.Tensor, r: int, world: int):
    """Gradients of :func:`prefix_state` with respect to every earlier rank's ``F_j`` and ``lP_j``:
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


class _StateExchange(torch.autograd.Function):
    """(F [nh,P,N], logP [nh]) of every rank -> the state entering this rank's slice."""

    @staticmethod
    def forward(ctx, F_local, logP, cp: ContextParallel, layer):
        nh = logP.shape[0]
        payload = torch.cat([F_local.reshape(-1).float(), logP.float()]).contiguous()
        recv = cp._exchange(payload, CH_STATE_F, +1, layer)
        ctx.layer = layer
        n = F_local.numel()
        Fs = recv[:, :n].view(cp.world, *F_local.shape)
        lPs = recv[:, n:].view(cp.world, nh)
        h = prefix_state(Fs, lPs, cp.rank) if cp.rank > 0 else torch.zeros_like(F_local, dtype=torch.float32)
        ctx.cp = cp
        ctx.save_for_backward(Fs[: cp.rank].clone(), lPs[: cp.rank].clone())
        return h

    @staticmethod
    def backward(ctx, dh):
        cp = ctx.cp
        Fs, lPs = ctx.saved_tensors
        r, nh = cp.rank, dh.shape[0]
        # local chain: H_r = sum_{j<r} (prod_{j<i<r} P_i) F_j ; gradients w.r.t. the F_j / logP_j of EARLIER ranks
        dF, dlP = prefix_state_grads(dh, Fs, lPs, r, cp.world)
        # send each earlier rank its share; collect what later ranks computed for THIS rank
        n = dh.numel()
        mine_F = torch.zeros_like(dh, dtype=torch.float32)
        mine_lP = torch.zeros(nh, dtype=torch.float32, device=dh.device)
        payload = torch.cat([dF.reshape(cp.world, -1), dlP], 1).contiguous()  # [world, n + nh], row j is for rank j
        recv = _exchange_rows(cp, payload, CH_STATE_B, -1, ctx.layer)         # [world(sender), n + nh]
        for s in range(r + 1, cp.world):
            mine_F += recv[s, :n].view_as(dh)
            mine_lP += recv[s, n:]
        return mine_F, mine_lP, None, None


def _exchange_rows(cp: ContextParallel, payload: torch.Tensor, chan: int, direction: int, tag=None) -> torch.Tensor:
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
                               direction, 1, epoch, st.data_ptr(), NV.stream_ptr())
    NV.check(rc, "fmsb_cp_push")
    rc = NV.lib().fmsb_cp_wait(cp.comm.signals.ptrs[cp.rank] + chan * cp.world * 4, cp.rank, cp.world, direction, 0, 0,
                               epoch, st.data_ptr(), NV.stream_ptr())
    NV.check(rc, "fmsb_cp_wait")
    return slots.buf.local.view(cp.world, slots.slot_bytes)[:, :nbytes].view(payload.dtype).view(cp.world, row)


class _HaloExchange(torch.autograd.Function):
    """Last ``k`` rows of the previous rank's conv input (zeros on rank 0)."""

    @staticmethod
    def forward(ctx, xBC, cp: ContextParallel, k: int, layer):
        tail = xBC[-k:].contiguous()
        recv = cp._exchange(tail.reshape(-1), CH_HALO_F, +1, layer)
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
        recv = _exchange_rows(cp, payload.contiguous(), CH_HALO_B + 4, -1, ctx.layer)
        dx = torch.zeros(ctx.shape, dtype=dhalo.dtype, device=dhalo.device)
        if cp.rank + 1 < cp.world:
            dx[-k:] = recv[cp.rank + 1].view(k, -1)
        return dx, None, None, None
