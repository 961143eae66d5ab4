"""Thread-level model of the peer-memory signalling protocols of ``csrc/comm.cu`` / ``csrc/moe.cu`` / ``csrc/cp.cu``.

One Python thread per rank; "symmetric memory" is a list of per-rank byte arrays every thread can address; signals
are per-rank ``[channel][world]`` epoch words.  The operations below follow the kernels step by step (same order of
payload stores, release of the signal, bounded acquire-wait, monotonically increasing epochs that are never reset,
double-buffered tables selected by epoch parity), so that slot reuse, epoch arithmetic and the time-out path can be
exercised, and faults injected (a dropped or delayed signal, a rank that stops), without a GPU.  Random scheduling
jitter is injected between every protocol step.
"""
from __future__ import annotations

import random
import threading
import time
from typing import Callable, Dict, List, Optional

import numpy as np

TIMEOUT_PEER_FLAG = 4  # same code as kTimeoutPeerFlag in csrc/common.cuh


class SimWorld:
    def __init__(self, world: int, channels: int = 8, jitter: float = 2e-4, wait_budget: float = 0.5, seed: int = 0):
        self.world, self.channels = world, channels
        self.signals = np.zeros((world, channels, world), dtype=np.int64)  # signals[owner][chan][writer]
        self.status = [0] * world
        self.jitter = jitter
        self.wait_budget = wait_budget
        self.buffers: Dict[str, List[np.ndarray]] = {}
        self.drop: Optional[Callable[[int, int, int, int], bool]] = None  # (writer, owner, chan, epoch) -> drop?
        self._rng = [random.Random(seed * 1000 + r) for r in range(world)]
        self._lock = threading.Lock()

    # -- symmetric allocations
    def alloc(self, name: str, n: int, dtype=np.float32) -> None:
        self.buffers[name] = [np.zeros(n, dtype=dtype) for _ in range(self.world)]

    # -- primitives
    def _pause(self, rank: int) -> None:
        if self.jitter:
            time.sleep(self._rng[rank].random() * self.jitter)

    def signal(self, writer: int, owner: int, chan: int, epoch: int) -> None:
        """st.release.sys of ``epoch`` into the owner's slot for ``writer``."""
        self._pause(writer)
        if self.drop is not None and self.drop(writer, owner, chan, epoch):
            return
        with self._lock:  # release: everything the writer stored before is visible once the word is
            self.signals[owner, chan, writer] = epoch

    def wait(self, rank: int, chan: int, writer: int, epoch: int) -> bool:
        """Bounded ld.acquire.sys spin until the slot reached ``epoch``; records the status code on expiry."""
        deadline = time.time() + self.wait_budget
        while True:
            with self._lock:
                seen = int(self.signals[rank, chan, writer])
            if seen - epoch >= 0:
                return True
            if self.status[rank] != 0 or time.time() > deadline:
                self.status[rank] = self.status[rank] or TIMEOUT_PEER_FLAG
                return False
            time.sleep(0)

    # -- protocols (each returns False when a wait ran out)
    def barrier(self, rank: int, chan: int, epoch: int) -> bool:
        for r in range(self.world):
            self.signal(rank, r, chan, epoch)
        return all(self.wait(rank, chan, r, epoch) for r in range(self.world))

    def allgather_pull(self, rank: int, src: str, dst: str, chan: int, epoch: int) -> bool:
        """shard of rank r = buffers[src][r]; every rank pulls all shards after a barrier that says they are written."""
        if not self.barrier(rank, chan, epoch):
            return False
        n = len(self.buffers[src][0])
        for r in range(self.world):
            self._pause(rank)
            self.buffers[dst][rank][r * n:(r + 1) * n] = self.buffers[src][r]
        return True

    def allreduce_two_shot(self, rank: int, bucket: str, chan: int, epoch: int) -> bool:
        """barrier -> reduce own slice from all peers (fp32, scaled) -> push result to every rank -> barrier."""
        if not self.barrier(rank, chan, epoch):
            return False
        n = len(self.buffers[bucket][0]) // self.world
        sl = slice(rank * n, (rank + 1) * n)
        acc = np.zeros(n, dtype=np.float64)
        for r in range(self.world):
            self._pause(rank)
            acc += self.buffers[bucket][r][sl]
        acc /= self.world
        # nobody may overwrite a slice that a peer has not finished reading: all reads of `sl` are done by its owner
        for r in range(self.world):
            self._pause(rank)
            self.buffers[bucket][r][sl] = acc
        return self.barrier(rank, chan + 1, epoch)

    def exchange_counts(self, rank: int, table: str, counts: np.ndarray, chan: int, epoch: int) -> Optional[np.ndarray]:
        """Expert-parallel plan: every rank pushes its per-destination counts into the peers' tables; tables are double
        buffered by epoch parity so that a fast rank's next step cannot overwrite what a slow rank still reads."""
        w = self.world
        half = len(self.buffers[table][0]) // 2
        base = (epoch & 1) * half
        for r in range(w):
            self._pause(rank)
            self.buffers[table][r][base + rank * w: base + (rank + 1) * w] = counts
        if not self.barrier(rank, chan, epoch):
            return None
        return self.buffers[table][rank][base: base + w * w].reshape(w, w).copy()

    def push_state(self, rank: int, slot: str, payload: np.ndarray, chan: int, epoch: int) -> None:
        """Context-parallel hand-off: write (state, decay) into every LATER rank's slot for this rank, then signal."""
        n = len(payload)
        for r in range(rank + 1, self.world):
            self._pause(rank)
            self.buffers[slot][r][rank * n:(rank + 1) * n] = payload
            self.signal(rank, r, chan, epoch)

    def wait_states(self, rank: int, slot: str, n: int, chan: int, epoch: int) -> Optional[np.ndarray]:
        for r in range(rank):
            if not self.wait(rank, chan, r, epoch):
                return None
        return self.buffers[slot][rank][: rank * n].reshape(rank, n).copy()


def run_ranks(world: SimWorld, fn: Callable[[int], None]) -> List[Optional[BaseException]]:
    """Run ``fn(rank)`` on one thread per rank; returns the exception (or None) of each."""
    errs: List[Optional[BaseException]] = [None] * world.world

    def body(r):
        try:
            fn(r)
        except BaseException as exc:  # noqa: BLE001
            errs[r] = exc

    threads = [threading.Thread(target=body, args=(r,)) for r in range(world.world)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    return errs
