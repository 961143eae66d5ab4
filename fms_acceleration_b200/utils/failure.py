"""Host-side failure detection between training steps.

The reference has none (a crashed rank shows up as an NCCL time-out in the others; the benchmark driver only
records tracebacks, scripts/benchmarks/benchmark.py:63-66).  Here every device-side wait is bounded and reports
through a status word, and the ranks additionally watch one another on the host, so that a rank that died, raised or
stalled is noticed *before* the next kernel that would wait for it is launched:

* each rank publishes ``(step, wall-clock time, state)`` in the job's key-value store after every step;
* before a step, :meth:`Heartbeat.check_peers` reads the peers' records and raises :class:`PeerFailure` when a peer
  reported a failure, left, or has not been heard from for ``stale_after`` seconds;
* :meth:`Heartbeat.guard` wraps a step: an exception inside it is published (state ``failed`` + message) before it
  propagates, so the survivors stop with a clear error instead of running into their wait budgets;
* :meth:`Heartbeat.rendezvous` is the host-side gate in front of a step's first collective.

The rank that hosts the store should be the last to exit after a failure (it lingers for a moment), otherwise the
others only learn that the store is gone.  The store is any ``torch.distributed`` store (TCPStore from the default process group, FileStore, HashStore); nothing
here touches a GPU, so the logic is tested with gloo ranks on the CPU.
"""
from __future__ import annotations

import contextlib
import json
import time
from typing import Dict, List, Optional

import torch.distributed as dist

ALIVE, FAILED, LEFT = "alive", "failed", "left"


class PeerFailure(RuntimeError):
    def __init__(self, rank: int, state: str, detail: str = ""):
        super().__init__(f"rank {rank} is {state}" + (f": {detail}" if detail else ""))
        self.rank, self.state, self.detail = rank, state, detail


class Heartbeat:
    def __init__(self, store, rank: int, world_size: int, stale_after: float = 60.0, prefix: str = "fmsb/hb"):
        self.store, self.rank, self.world = store, rank, world_size
        self.stale_after = stale_after
        self.prefix = prefix
        self.step = 0
        self._publish(ALIVE)

    @classmethod
    def from_default_group(cls, stale_after: float = 60.0) -> "Heartbeat":
        from torch.distributed.distributed_c10d import _get_default_store

        return cls(_get_default_store(), dist.get_rank(), dist.get_world_size(), stale_after)

    def _key(self, rank: int) -> str:
        return f"{self.prefix}/{rank}"

    def _publish(self, state: str, detail: str = "") -> None:
        rec = {"step": self.step, "time": time.time(), "state": state, "detail": detail[:500]}
        self.store.set(self._key(self.rank), json.dumps(rec))

    def beat(self, step: Optional[int] = None) -> None:
        self.step = self.step + 1 if step is None else step
        self._publish(ALIVE)

    def leave(self) -> None:
        """Orderly exit between steps (no kernel or collective of this rank in flight)."""
        self._publish(LEFT)

    def fail(self, detail: str) -> None:
        self._publish(FAILED, detail)

    def peers(self) -> Dict[int, dict]:
        out = {}
        for r in range(self.world):
            if r == self.rank:
                continue
            try:
                if hasattr(self.store, "check") and not self.store.check([self._key(r)]):
                    continue  # the peer has not started yet
                out[r] = json.loads(self.store.get(self._key(r)).decode())
            except (ValueError, KeyError):
                continue
            except RuntimeError as exc:
                # the store itself is gone: the rank that hosts it (rank 0 for the default TCP store) has exited
                raise PeerFailure(0, "unreachable", f"key-value store does not answer ({exc})".splitlines()[0]) from exc
        return out

    def check_peers(self) -> None:
        now = time.time()
        for r, rec in sorted(self.peers().items()):
            if rec["state"] in (FAILED, LEFT):
                raise PeerFailure(r, rec["state"], rec.get("detail", ""))
            if now - rec["time"] > self.stale_after:
                raise PeerFailure(r, "stale", f"no heartbeat for {now - rec['time']:.1f} s (last step {rec['step']})")

    def wait_for_peers(self, step: int, timeout: float, poll: float = 0.02) -> None:
        """Host-side rendezvous: return when every peer reached ``step``; raise as soon as one failed or left, or when
        ``timeout`` runs out (then naming the slowest peer)."""
        deadline = time.time() + timeout
        while True:
            recs = self.peers()
            behind: List[int] = []
            for r in range(self.world):
                if r == self.rank:
                    continue
                rec = recs.get(r)
                if rec is None:
                    behind.append(r)
                    continue
                if rec["state"] in (FAILED, LEFT) and rec["step"] < step:
                    raise PeerFailure(r, rec["state"], rec.get("detail", ""))
                if rec["step"] < step:
                    behind.append(r)
            if not behind:
                return
            if time.time() > deadline:
                raise PeerFailure(behind[0], "stale", f"did not reach step {step} within {timeout} s")
            time.sleep(poll)

    def rendezvous(self, step: int, timeout: float) -> None:
        """Announce that this rank is about to run the kernels / collectives of ``step`` and wait until every peer
        announced the same.  A peer that failed or left before announcing ``step`` ends the wait with
        :class:`PeerFailure`, so nothing that would wait for it on the device gets launched."""
        self.beat(step)
        self.wait_for_peers(step, timeout)

    @contextlib.contextmanager
    def guard(self):
        """``with hb.guard(): step()`` - check the peers first; an exception in the body is published before it
        propagates."""
        self.check_peers()
        try:
            yield
        except BaseException as exc:  # noqa: BLE001 - the point is to tell the others, then re-raise
            self.fail(f"{type(exc).__name__}: {exc}")
            raise
