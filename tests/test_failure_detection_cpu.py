"""Failure detection without a GPU: protocol model on threads (dropped signals, stopped ranks, slot reuse) and the
host heartbeat between gloo ranks (a rank that raises, a rank that leaves, a rank that never joins)."""
import os
import subprocess
import sys
import textwrap

import numpy as np
import pytest

from fms_acceleration_b200.utils.failure import Heartbeat, PeerFailure
from fms_acceleration_b200.utils.protocol_sim import TIMEOUT_PEER_FLAG, SimWorld, run_ranks


# ------------------------------------------------------------------------------------------- protocol model
@pytest.mark.parametrize("world", [2, 4, 8])
def test_allreduce_and_allgather_many_epochs(world):
    sim = SimWorld(world, seed=world)
    n = 16 * world
    sim.alloc("bucket", n, np.float64)
    sim.alloc("shard", 8, np.float64)
    sim.alloc("full", 8 * world, np.float64)
    steps = 12
    results = [[None] * steps for _ in range(world)]

    def rank_fn(r):
        rng = np.random.default_rng(r)
        for step in range(1, steps + 1):
            sim.buffers["bucket"][r][:] = rng.standard_normal(n) + step
            assert sim.allreduce_two_shot(r, "bucket", 0, step)
            results[r][step - 1] = sim.buffers["bucket"][r].copy()
            sim.buffers["shard"][r][:] = r * 100 + step
            assert sim.allgather_pull(r, "shard", "full", 2, step)
            assert np.array_equal(sim.buffers["full"][r], np.repeat(np.arange(world) * 100 + step, 8))
            assert sim.barrier(r, 3, step)  # shards may be rewritten only after everybody pulled

    errs = run_ranks(sim, rank_fn)
    assert errs == [None] * world, errs
    for step in range(steps):
        for r in range(1, world):
            assert np.allclose(results[r][step], results[0][step])  # every rank holds the same average
    assert sim.status == [0] * world


def test_double_buffered_count_tables_survive_a_fast_rank():
    world = 4
    sim = SimWorld(world, jitter=5e-4, seed=3)
    sim.alloc("table", 2 * world * world, np.int64)
    seen = [[] for _ in range(world)]

    def rank_fn(r):
        for step in range(1, 9):
            counts = np.arange(world) + 10 * r + 100 * step
            t = sim.exchange_counts(r, "table", counts, 0, step)
            assert t is not None
            seen[r].append(t)

    assert run_ranks(sim, rank_fn) == [None] * world
    for step in range(8):
        expect = np.stack([np.arange(world) + 10 * r + 100 * (step + 1) for r in range(world)])
        for r in range(world):
            assert np.array_equal(seen[r][step], expect)


def test_single_dropped_signal_heals_with_the_next_epoch():
    """Waits compare with >=, so a lost epoch-3 word is covered by the epoch-4 word of the same writer."""
    world = 4
    sim = SimWorld(world, wait_budget=2.0)
    sim.drop = lambda writer, owner, chan, epoch: writer == 2 and owner == 0 and epoch == 3
    ok = [[] for _ in range(world)]

    def rank_fn(r):
        for step in range(1, 6):
            ok[r].append(sim.barrier(r, 0, step))

    run_ranks(sim, rank_fn)
    assert all(o == [True] * 5 for o in ok) and sim.status == [0] * world


def test_lost_link_times_out_with_status_instead_of_hanging():
    world = 4
    sim = SimWorld(world, wait_budget=0.2)
    sim.drop = lambda writer, owner, chan, epoch: writer == 2 and owner == 0 and epoch >= 3
    ok = [[] for _ in range(world)]

    def rank_fn(r):
        for step in range(1, 5):
            good = sim.barrier(r, 0, step)
            ok[r].append(good)
            if not good:
                return

    run_ranks(sim, rank_fn)
    assert ok[0] == [True, True, False]  # rank 0 never hears from rank 2 again
    assert sim.status[0] == TIMEOUT_PEER_FLAG
    # the others passed barrier 3 (they got all signals) and ran out at barrier 4, where rank 0 no longer takes part
    assert all(o[:3] == [True, True, True] and o[3] is False for o in ok[1:])


@pytest.mark.parametrize("world,chunks", [(2, 2), (3, 5), (4, 3)])
def test_staged_expert_exchange_reuses_its_two_staging_sets_safely(world, chunks):
    """The chunk-pipelined expert-parallel exchange (two streams per rank, two staging sets) under scheduling
    jitter: every row comes back right, call after call (the sets and the epochs are reused across calls)."""
    from fms_acceleration_b200.utils.protocol_sim import StagedExchange

    sim = SimWorld(world, jitter=3e-4, wait_budget=5.0, seed=3)
    for _ in range(3):
        ex = StagedExchange(sim, chunks, rows=4)
        # epochs continue across calls, as they do across layers
        ex.epoch = getattr(sim, "_ep_epochs", ex.epoch)
        assert ex.run()
        sim._ep_epochs = ex.epoch
    assert sim.status == [0] * world


def test_staged_expert_exchange_model_catches_a_single_staging_set():
    """With ONE staging set, chunk c+1 is pushed while a slower owner may not have copied chunk c out yet: the bug
    the second set prevents.  The model must see corrupted rows then (or the test above proves nothing)."""
    from fms_acceleration_b200.utils.protocol_sim import StagedExchange

    bad = 0
    for seed in range(8):
        sim = SimWorld(3, jitter=2e-3, wait_budget=5.0, seed=seed)
        if not StagedExchange(sim, 6, rows=4, sets=1).run():
            bad += 1
    assert bad > 0


def test_staged_expert_exchange_dropped_barrier_signal_times_out():
    """One barrier signal of one chunk never arrives: the waiting ranks give up with the peer-flag status and every
    thread returns (nothing hangs, nothing reads half-written rows as results)."""
    from fms_acceleration_b200.utils.protocol_sim import StagedExchange

    sim = SimWorld(3, jitter=1e-4, wait_budget=0.3, seed=1)
    sim.drop = lambda writer, owner, chan, epoch: (writer, owner, chan, epoch) == (1, 2, StagedExchange.CH_A, 2)
    ex = StagedExchange(sim, 4, rows=4)
    assert ex.run() is False
    assert sim.status[2] == TIMEOUT_PEER_FLAG


def test_context_parallel_handoff_order():
    world, n = 4, 6
    sim = SimWorld(world, seed=5)
    sim.alloc("slot", world * n, np.float64)
    got = [None] * world

    def rank_fn(r):
        for step in (1, 2, 3):
            sim.push_state(r, "slot", np.full(n, 10.0 * r + step), 0, step)
            st = sim.wait_states(r, "slot", n, 0, step)
            assert st is not None
            got[r] = st
            assert sim.barrier(r, 1, step)  # slots are per layer on the GPU; here one slot, so fence the reuse

    assert run_ranks(sim, rank_fn) == [None] * world
    assert got[0].shape == (0, n)
    assert np.array_equal(got[3], np.stack([np.full(n, 10.0 * r + 3) for r in range(3)]))


# ------------------------------------------------------------------------------------------- heartbeat
def test_heartbeat_with_a_hash_store():
    import torch.distributed as dist

    store = dist.HashStore()
    a, b = Heartbeat(store, 0, 2, stale_after=0.3), Heartbeat(store, 1, 2, stale_after=0.3)
    a.check_peers()
    with a.guard():
        a.beat()
    assert a.step == 1
    with pytest.raises(ValueError):
        with b.guard():
            raise ValueError("boom on rank 1")
    with pytest.raises(PeerFailure, match="rank 1 is failed: ValueError: boom"):
        a.check_peers()
    b.beat()
    a.check_peers()
    import time

    time.sleep(0.4)
    with pytest.raises(PeerFailure, match="stale"):
        a.check_peers()
    b.leave()
    with pytest.raises(PeerFailure, match="left"):
        a.wait_for_peers(5, timeout=1.0)


WORKER = textwrap.dedent("""
    import os, sys, time, datetime
    import torch, torch.distributed as dist
    sys.path.insert(0, os.environ["REPO"])
    from fms_acceleration_b200.utils.failure import Heartbeat, PeerFailure
    mode = os.environ["MODE"]
    dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=20))
    rank, world = dist.get_rank(), dist.get_world_size()
    hb = Heartbeat.from_default_group(stale_after=5.0)
    x = torch.ones(4)
    try:
        for step in range(1, 6):
            with hb.guard():
                if mode == "raise" and rank == 1 and step == 3:
                    raise RuntimeError("injected failure in step 3")
                if mode == "leave" and rank == 1 and step == 3:
                    hb.leave()
                    print("rank 1 left between steps", flush=True)
                    os._exit(0)
                hb.rendezvous(step, timeout=10.0)   # the host learns of a failure BEFORE the collective
                dist.all_reduce(x)
        print(f"rank {rank} finished", flush=True)
    except PeerFailure as exc:
        print(f"rank {rank} stopped cleanly: {exc}", flush=True)
        if rank == 0:
            time.sleep(1.5)   # host of the store: let the others read the failure record first
        os._exit(3)
    except RuntimeError as exc:
        print(f"rank {rank} raised: {exc}", flush=True)
        os._exit(4)
""")


@pytest.mark.parametrize("mode,codes", [("ok", {0}), ("raise", {3, 4}), ("leave", {0, 3})])
def test_gloo_ranks_notice_a_failed_peer_between_steps(tmp_path, mode, codes):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    port = 29600 + (os.getpid() + len(mode)) % 300
    procs = []
    for r in range(3):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE="3", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), MODE=mode,
                   REPO=repo)
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    outs = []
    for p in procs:
        out, _ = p.communicate(timeout=120)  # a hang here is the failure this test exists to catch
        outs.append(out)
    got = {p.returncode for p in procs}
    assert got == codes, outs
    if mode == "raise":
        assert "rank 1 raised: injected failure" in outs[1]
        assert all("stopped cleanly: rank 1 is failed" in outs[r] for r in (0, 2)), outs
    if mode == "leave":
        assert all("stopped cleanly: rank 1 is left" in outs[r] for r in (0, 2)), outs


def test_rank_that_never_joins_ends_the_rendezvous_with_an_error(tmp_path):
    script = tmp_path / "w.py"
    script.write_text(textwrap.dedent("""
        import datetime, sys, torch.distributed as dist
        try:
            dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=3))
        except Exception as exc:
            print("rendezvous failed:", type(exc).__name__, flush=True)
            sys.exit(5)
    """))
    env = dict(os.environ, RANK="0", WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(29950 + os.getpid() % 40))
    p = subprocess.run([sys.executable, str(script)], env=env, capture_output=True, text=True, timeout=90)
    assert p.returncode == 5 and "rendezvous failed" in p.stdout
