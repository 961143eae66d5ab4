"""Symmetric memory: buffers that every rank of a process group allocates identically and whose peer copies
can be addressed directly from kernels.

Bootstrap uses ``torch.distributed._symmetric_memory`` (CUDA virtual-memory handles exchanged through the
process group's store); everything that moves data afterwards is this package's own kernels
(``csrc/comm.cu`` and the fused compute+communication kernels), which receive the table of peer addresses.
"""
from __future__ import annotations

import ctypes
import os
from typing import List, Optional

import torch
import torch.distributed as dist

from .. import _native as N

P, I, L, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
U = ctypes.c_uint
N.declare("fmsb_comm_barrier", [P, I, I, I, U, P, P])
N.declare("fmsb_comm_allgather", [P, P, L, I, I, I, P])
N.declare("fmsb_comm_reduce_scatter", [P, P, L, I, I, F, I, I, I, P])
N.declare("fmsb_comm_allreduce", [P, P, L, I, I, F, I, I, U, P, I, P, P])
N.declare("fmsb_comm_wait_flag", [P, U, P, L, P])
N.declare("fmsb_comm_allreduce_multimem", [P, P, L, I, I, F, I, I, U, P, I, P, P])

N_CHANNELS = 64


def _ptr_array(ptrs: List[int]):
    arr = (ctypes.c_void_p * len(ptrs))(*ptrs)
    return arr


class SymmBuffer:
    """One symmetric allocation of ``nbytes`` (uint8) per rank."""

    def __init__(self, nbytes: int, group: Optional[dist.ProcessGroup] = None, device=None, zero: bool = True):
        import torch.distributed._symmetric_memory as symm_mem

        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        nbytes = (int(nbytes) + 255) // 256 * 256
        self.nbytes = nbytes
        self.local = symm_mem.empty(nbytes, dtype=torch.uint8, device=device)
        if zero:
            self.local.zero_()
        self.handle = symm_mem.rendezvous(self.local, self.group)
        self.ptrs: List[int] = [int(p) for p in self.handle.buffer_ptrs]
        self._arr = _ptr_array(self.ptrs)
        # address of the NVSwitch multicast object the allocation is bound to (0 where the fabric offers none):
        # multimem loads / stores on it reach every rank's copy through the switch
        self.mc_ptr: int = int(getattr(self.handle, "multicast_ptr", 0) or 0)

    def ptr_array(self, offset: int = 0):
        """ctypes array of the peers' base addresses (+ ``offset`` bytes)."""
        if offset == 0:
            return self._arr
        return _ptr_array([p + offset for p in self.ptrs])

    def ptr_array_strided(self, offset: int, stride: int):
        """ctypes array whose entry r is rank r's base address + ``offset`` + r * ``stride`` bytes."""
        return _ptr_array([p + offset + r * stride for r, p in enumerate(self.ptrs)])

    def view(self, offset: int, numel: int, dtype: torch.dtype) -> torch.Tensor:
        nb = numel * torch.empty((), dtype=dtype).element_size()
        return self.local[offset: offset + nb].view(dtype)


class Communicator:
    """Signal words, epochs and the peer-memory collectives of one process group."""

    def __init__(self, group: Optional[dist.ProcessGroup] = None, device=None):
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.signals = SymmBuffer(N_CHANNELS * self.world * 4, self.group, self.device)
        self.grid_sync = torch.zeros(8, dtype=torch.int32, device=self.device)
        self.epochs = [0] * N_CHANNELS
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)

    def next_epoch(self, chan: int) -> int:
        self.epochs[chan] += 1
        return self.epochs[chan]

    # ------------------------------------------------------------------ collectives
    def barrier(self, chan: int = 0) -> None:
        """Device-side barrier on the current stream (no host synchronisation)."""
        st = N.status_word(self.device)
        rc = N.lib().fmsb_comm_barrier(self.signals.ptr_array(), self.rank, self.world, chan, self.next_epoch(chan),
                                       st.data_ptr(), N.stream_ptr())
        N.check(rc, "fmsb_comm_barrier")

    def allgather_into(self, shards: SymmBuffer, shard_offset: int, shard_bytes: int, dst: torch.Tensor,
                       ctas: int = 32) -> None:
        """dst[r*shard_bytes:(r+1)*shard_bytes] <- bytes [shard_offset, +shard_bytes) of rank r's ``shards``."""
        assert dst.numel() * dst.element_size() >= shard_bytes * self.world
        rc = N.lib().fmsb_comm_allgather(shards.ptr_array(shard_offset), dst.data_ptr(), shard_bytes, self.rank,
                                         self.world, ctas, N.stream_ptr())
        N.check(rc, "fmsb_comm_allgather")

    def allreduce_(self, bucket: SymmBuffer, numel: int, dtype: torch.dtype, scale: Optional[float] = None,
                   chan: int = 2, ctas: Optional[int] = None, multimem: Optional[bool] = None) -> None:
        self.allreduce_ptrs(bucket.ptr_array(), numel, dtype, scale, chan, ctas, mc_ptr=bucket.mc_ptr, multimem=multimem)

    def allreduce_ptrs(self, ptrs, numel: int, dtype: torch.dtype, scale: Optional[float] = None,
                       chan: int = 2, ctas: Optional[int] = None, mc_ptr: int = 0,
                       multimem: Optional[bool] = None) -> None:
        """In-place sum (times ``scale``, default 1/world) of the first ``numel`` elements of a symmetric bucket.
        ``ctas`` defaults to 32 for adapter-sized buckets and to 128 for buckets of 32 MiB and more (a full
        fine-tune's gradients), which runs at the end of the backward when nothing else needs the SMs."""
        if ctas is None:
            nbytes = numel * torch.empty((), dtype=dtype).element_size()
            ctas = 32 if nbytes < (32 << 20) else 128
        st = N.status_word(self.device)
        scale = 1.0 / self.world if scale is None else scale
        self.epochs[chan + 1] = self.epochs[chan] + 1
        if multimem is None:
            multimem = os.environ.get("FMSB_ALLREDUCE", "p2p") == "multimem"
        if multimem and mc_ptr and dtype in (torch.bfloat16, torch.float32):
            # in-switch reduction (NVLS): one multimem load returns the sum over the ranks, one multimem store
            # writes the result everywhere
            rc = N.lib().fmsb_comm_allreduce_multimem(mc_ptr, self.signals.ptr_array(), numel, self.rank, self.world,
                                                      float(scale), N.dtype_code(dtype), chan, self.next_epoch(chan),
                                                      self.grid_sync.data_ptr(), ctas, st.data_ptr(), N.stream_ptr())
            N.check(rc, "fmsb_comm_allreduce_multimem")
            return
        rc = N.lib().fmsb_comm_allreduce(ptrs, self.signals.ptr_array(), numel, self.rank, self.world,
                                         float(scale), N.dtype_code(dtype), chan, self.next_epoch(chan),
                                         self.grid_sync.data_ptr(), ctas, st.data_ptr(), N.stream_ptr())
        N.check(rc, "fmsb_comm_allreduce")

    def reduce_scatter(self, bucket: SymmBuffer, n_own: int, dtype: torch.dtype, out: torch.Tensor,
                       scale: Optional[float] = None, chan: int = 4, ctas: int = 64) -> None:
        """out[n_own] <- scale * sum over ranks of their bucket slice owned by this rank (barriers included)."""
        self.reduce_scatter_ptrs(bucket.ptr_array(), n_own, dtype, out, scale, chan, ctas)

    def reduce_scatter_ptrs(self, ptrs, n_own: int, dtype: torch.dtype, out: torch.Tensor,
                            scale: Optional[float] = None, chan: int = 4, ctas: int = 64) -> None:
        """The same on a window of the peers' buffers: ``ptrs[r]`` is where rank r's world * n_own elements start."""
        scale = 1.0 / self.world if scale is None else scale
        self.barrier(chan)
        rc = N.lib().fmsb_comm_reduce_scatter(ptrs, out.data_ptr(), n_own, self.rank, self.world,
                                              float(scale), N.dtype_code(dtype), int(out.dtype == torch.float32),
                                              ctas, N.stream_ptr())
        N.check(rc, "fmsb_comm_reduce_scatter")
        self.barrier(chan + 1)
