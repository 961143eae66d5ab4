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


class StagedExchange:
    """The chunk-pipelined expert-parallel exchange of ``ops/moe.py`` with its two streams per rank.

    Every rank runs two threads: the *communication stream* (push rows into the owners' staging set, barrier, copy
    them out; later reduce the results into the staging set, barrier, read them back) and the *compute stream* (the
    experts).  Events order the two inside a rank exactly as the CUDA events do; the barriers are the cross-rank
    epoch barriers.  Two staging sets are reused every other chunk.  What must hold: a set is never overwritten
    while an owner still copies it out or a source still reads results from it.  The payload makes a violation
    visible: row values encode (source, chunk, index) and the "expert" maps ``x -> 2 x + owner``.

    ``sets``: number of staging sets, 2 (what the code does) or 1 (chunk c+1 is pushed into the set an owner may not
    have copied chunk c out of yet: the reuse bug that the second set prevents; the model must catch it)."""

    CH_A, CH_B = 0, 1

    def __init__(self, sim: SimWorld, n_chunks: int, rows: int, sets: int = 2):
        self.sim, self.C, self.rows, self.sets = sim, n_chunks, rows, sets
        w = sim.world
        sim.alloc("stage_x", 2 * w * rows, np.float64)   # [set][source][row]
        sim.alloc("stage_y", 2 * w * rows, np.float64)
        self.epoch = [[0, 0] for _ in range(w)]
        self.ready = [[threading.Event() for _ in range(n_chunks)] for _ in range(w)]
        self.done = [[threading.Event() for _ in range(n_chunks)] for _ in range(w)]
        self.xs = [[None] * n_chunks for _ in range(w)]
        self.ys = [[None] * n_chunks for _ in range(w)]
        self.out = [[None] * n_chunks for _ in range(w)]
        self.failed = [False] * w

    @staticmethod
    def value(src: int, chunk: int, i: int) -> float:
        return 1000.0 * src + 10.0 * chunk + 0.001 * i

    def _barrier(self, rank: int, chan: int) -> bool:
        self.epoch[rank][chan] += 1
        return self.sim.barrier(rank, chan, self.epoch[rank][chan])

    def _push(self, rank: int, c: int) -> bool:
        sim, w, n, s = self.sim, self.sim.world, self.rows, c % self.sets
        payload = np.array([self.value(rank, c, i) for i in range(n)])
        for owner in range(w):  # every owner gets this source's rows (one per (token, rank))
            sim._pause(rank)
            base = (s * w + rank) * n
            sim.buffers["stage_x"][owner][base: base + n] = payload
        if not self._barrier(rank, self.CH_A):
            return False
        sim._pause(rank)
        self.xs[rank][c] = sim.buffers["stage_x"][rank][s * w * n: (s + 1) * w * n].copy()  # replicate (local)
        self.ready[rank][c].set()
        return True

    def _pull(self, rank: int, c: int) -> bool:
        sim, w, n, s = self.sim, self.sim.world, self.rows, c % self.sets
        if not self.done[rank][c].wait(timeout=10 * sim.wait_budget + 5):
            return False
        sim._pause(rank)
        sim.buffers["stage_y"][rank][s * w * n: (s + 1) * w * n] = self.ys[rank][c]        # owner-side reduction
        if not self._barrier(rank, self.CH_B):
            return False
        got = np.zeros(n)
        for owner in range(w):  # one row per (token, owner) comes back
            sim._pause(rank)
            base = (s * w + rank) * n
            got += sim.buffers["stage_y"][owner][base: base + n]
        self.out[rank][c] = got
        return True

    def comm_stream(self, rank: int) -> None:
        C = self.C
        ok = self._push(rank, 0) and (C < 2 or self._push(rank, 1))
        for c in range(C):
            if not ok:
                break
            ok = self._pull(rank, c) and (c + 2 >= C or self._push(rank, c + 2))
        if not ok:
            self.failed[rank] = True
            for ev in self.ready[rank] + self.done[rank]:
                ev.set()  # let the other stream of this rank unwind

    def compute_stream(self, rank: int) -> None:
        for c in range(self.C):
            self.ready[rank][c].wait()
            if self.failed[rank]:
                return
            self.sim._pause(rank)
            self.ys[rank][c] = 2.0 * self.xs[rank][c] + rank
            self.done[rank][c].set()

    def expected(self, rank: int, c: int) -> np.ndarray:
        w = self.sim.world
        x = np.array([self.value(rank, c, i) for i in range(self.rows)])
        return sum(2.0 * x + owner for owner in range(w))

    def run(self) -> bool:
        """Returns True when every rank got every chunk right; False on a time-out (status set) or wrong data."""
        w = self.sim.world
        threads = [threading.Thread(target=self.comm_stream, args=(r,)) for r in range(w)]
        threads += [threading.Thread(target=self.compute_stream, args=(r,)) for r in range(w)]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        if any(self.failed):
            return False
        return all(self.out[r][c] is not None and np.allclose(self.out[r][c], self.expected(r, c))
                   for r in range(w) for c in range(self.C))


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
