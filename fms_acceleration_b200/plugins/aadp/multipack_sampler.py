"""Multipack distributed batch sampler: every step, all ranks receive batches with (nearly) the same number of
tokens, which removes the straggler effect of length-imbalanced data-parallel batches.

Interface and semantics of fms_acceleration_aadp/multipack_sampler.py:398-485 in the reference
(``MultipackDistributedBatchSampler(batch_max_length, lengths, num_replicas, rank, seed, padding)``, per-epoch
seeded permutation, samples longer than the capacity dropped with a warning, efficiency counters).  The
allocator itself is compiled C++ (``csrc/multipack.cpp``) instead of numba; a NumPy implementation of the same
algorithm is kept as the oracle and as the fallback when the native library has not been built.
"""
from __future__ import annotations

import ctypes
import warnings
from typing import List, Optional

import numpy as np
import torch.distributed as dist
from torch.utils.data import Sampler

from ... import _native as N

N.declare("fmsb_multipack_allocate", [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_longlong, ctypes.c_int,
                                      ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p])


# ------------------------------------------------------------------------------------------- NumPy oracle
def _fits(a: np.ndarray, c: int, n: int, padding: bool) -> bool:
    a = np.sort(a)[::-1]
    if not padding:
        free = np.full(n, c, dtype=np.int64)
        for s in a:
            ok = np.nonzero(free >= s)[0]
            if ok.size == 0:
                return False
            free[ok[0]] -= s
        return True
    longest = np.zeros(n, dtype=np.int64)
    cnt = np.zeros(n, dtype=np.int64)
    for s in a:
        cand = np.maximum(longest, s) * (cnt + 1)
        ok = np.nonzero(cand <= c)[0]
        if ok.size == 0:
            return False
        b = ok[0]
        longest[b] = max(longest[b], s)
        cnt[b] += 1
    return True


def _assign(a: np.ndarray, c: int, start: int, padding: bool) -> List[List[int]]:
    order = np.argsort(-a, kind="stable")
    bins: List[List[int]] = []
    state: List[int] = []
    cnt: List[int] = []
    for i in order:
        s = int(a[i])
        placed = False
        for b in range(len(bins)):
            if not padding:
                if state[b] >= s:
                    state[b] -= s
                    bins[b].append(start + int(i))
                    placed = True
                    break
            else:
                longest = max(state[b], s)
                if longest * (cnt[b] + 1) <= c:
                    state[b] = longest
                    cnt[b] += 1
                    bins[b].append(start + int(i))
                    placed = True
                    break
        if not placed:
            bins.append([start + int(i)])
            state.append(s if padding else c - s)
            cnt.append(1)
    return bins


def allocate_reference(lengths: np.ndarray, rank: int, c: int, n: int, padding: bool):
    """Pure NumPy version of the allocator (see ``csrc/multipack.cpp`` for the algorithm)."""
    cumsum = np.cumsum(lengths)
    start, consumed, out = 0, 0, []
    while True:
        upto = int(np.searchsorted(cumsum[start:], consumed + c * n, side="right"))
        lo, hi = 1, 1 + upto
        while hi - lo > 1:
            mid = (lo + hi) // 2
            if _fits(lengths[start: start + mid], c, n, padding):
                lo = mid
            else:
                hi = mid
        take = min(lo, len(lengths) - start)
        bins = _assign(lengths[start: start + take], c, start, padding)
        if len(bins) < n:
            break
        start += take
        consumed = int(cumsum[start - 1])
        out.append(bins[rank])
    return out, consumed, len(out) * c * n


def allocate(lengths: np.ndarray, lengths_cumsum: Optional[np.ndarray], rank: int, c: int, n: int, padding: bool = True):
    """Returns ``(batches, tokens_used, token_slots)``; batches are lists of positions into ``lengths``."""
    lengths = np.ascontiguousarray(lengths, dtype=np.int64)
    c = int(c)
    if not N.available():
        return allocate_reference(lengths, rank, c, n, padding)
    count = len(lengths)
    idx = np.empty(max(count, 1), dtype=np.int64)
    off = np.empty(count + 1, dtype=np.int64)
    stats = np.zeros(3, dtype=np.int64)
    rc = N.lib().fmsb_multipack_allocate(lengths.ctypes.data, count, rank, c, n, int(padding), idx.ctypes.data,
                                         off.ctypes.data, stats.ctypes.data)
    N.check(rc, "fmsb_multipack_allocate")
    nb = int(stats[0])
    batches = [idx[off[b]: off[b + 1]].tolist() for b in range(nb)]
    return batches, int(stats[1]), int(stats[2])


class MultipackDistributedBatchSampler(Sampler):
    def __init__(self, batch_max_length: int, lengths, num_replicas: Optional[int] = None, rank: Optional[int] = None,
                 seed: int = 0, padding: bool = True):
        if num_replicas is None:
            if not (dist.is_available() and dist.is_initialized()):
                raise RuntimeError("Requires distributed package to be available")
            num_replicas = dist.get_world_size()
        if rank is None:
            if not (dist.is_available() and dist.is_initialized()):
                raise RuntimeError("Requires distributed package to be available")
            rank = dist.get_rank()
        assert isinstance(lengths, np.ndarray), "lengths must be a numpy array"
        self.num_replicas, self.rank, self.seed = num_replicas, rank, seed
        self.batch_max_length = batch_max_length
        self.lengths = lengths
        self.padding = padding
        self.epoch = 0
        self.eff_total_used = 0
        self.eff_total_slots = 0

    def set_epoch(self, epoch: int) -> None:
        self.epoch = epoch

    def generate_batches(self, set_stats: bool = False):
        order = np.random.default_rng(seed=self.seed + self.epoch).permutation(len(self.lengths))
        keep = order[self.lengths[order] <= self.batch_max_length]
        if len(keep) < len(self.lengths):
            warnings.warn(f"Dropping {len(self.lengths) - len(keep)} samples longer than batch_max_length. "
                          "Ensure that the right max_batch_length is used during data processing.")
        lengths = self.lengths[keep]
        batches, used, slots = allocate(lengths, None, self.rank, int(self.batch_max_length), self.num_replicas,
                                        self.padding)
        batches = [keep[np.asarray(b, dtype=np.int64)] for b in batches]
        if set_stats:
            self.eff_total_used += used
            self.eff_total_slots += slots
        return batches

    def __iter__(self):
        return iter(self.generate_batches(set_stats=True))

    def num_batches(self) -> int:
        return len(self.generate_batches())

    def __len__(self) -> int:
        return self.num_batches()

    def efficiency(self) -> float:
        return self.eff_total_used / max(self.eff_total_slots, 1)


# ------------------------------------------------------------------------------------------- batch-size helpers
def find_max_pack_len_with_padding(lengths: np.ndarray, samples_per_minibatch: int, num_gpus: int,
                                   avg_sample_len: float, seed: int = 0) -> int:
    """Largest per-GPU token capacity (searched in steps of 20 above the average) for which a padded multipack
    epoch still yields at least ``samples_per_minibatch`` samples per step on average."""
    def samples_per_step(cap: int) -> float:
        s = MultipackDistributedBatchSampler(cap, lengths, num_gpus, 0, seed, padding=True)
        b = s.generate_batches()
        return (len(lengths) / max(len(b), 1)) if b else 0.0

    base = int(avg_sample_len * samples_per_minibatch / num_gpus)
    add = 0
    while samples_per_step(base + add) < samples_per_minibatch and add < 20 * 1000:
        add += 20
    return base + add


def find_packing_max_batch_len_and_grad_accum(num_gpus: int, avg_sample_len: float, effective_batch_size: int,
                                              max_batch_len_per_gpu: int, is_padding: bool = False,
                                              dataset_lengths: Optional[np.ndarray] = None, seed: int = 0):
    """Smallest gradient-accumulation count for which the per-GPU token capacity stays within
    ``max_batch_len_per_gpu``; returns ``(packing_max_batch_len, grad_accum)``."""
    grad_accum = 0
    cap = max_batch_len_per_gpu + 1
    while cap > max_batch_len_per_gpu:
        grad_accum += 1
        per_step = effective_batch_size / grad_accum
        if is_padding and dataset_lengths is not None:
            cap = find_max_pack_len_with_padding(dataset_lengths, int(per_step), num_gpus, avg_sample_len, seed)
        else:
            cap = int(avg_sample_len * per_step / num_gpus)
    return cap, grad_accum


# ------------------------------------------------------------------------------------------- reference-named helpers
# The reference exposes its packing primitives and its padded-capacity search as module-level functions
# (fms_acceleration_aadp/multipack_sampler.py:38-164, 230-340); the same names here, on top of this module's allocator.
def ffd_check(a: np.ndarray, c: int, n: int) -> bool:
    """Do the lengths ``a`` fit into ``n`` bins of ``c`` tokens (first-fit decreasing)?"""
    return _fits(np.asarray(a), int(c), int(n), False)


def ffd_check_padding(a: np.ndarray, c: int, n: int) -> bool:
    """The same when every bin is padded to its longest sample (a bin costs ``longest x samples``)."""
    return _fits(np.asarray(a), int(c), int(n), True)


def ffd_with_result(a: np.ndarray, c: int, start_index: int) -> List[List[int]]:
    """First-fit-decreasing bins of capacity ``c`` as lists of ``start_index + position``."""
    return _assign(np.asarray(a), int(c), int(start_index), False)


def ffd_with_result_padding(a: np.ndarray, c: int, start_index: int) -> List[List[int]]:
    return _assign(np.asarray(a), int(c), int(start_index), True)


def _padded_capacity(base_avg: float, addition: float, goal: int, num_gpus: int, grad_accum: int) -> int:
    return int((base_avg + addition) * ((goal / num_gpus) / grad_accum))


def guess_starting_avg_padding(base_avg, goal, num_gpus, grad_accum, sorted_lengths) -> int:
    """Average padding per sample of the first bucket that the longest samples would form (``sorted_lengths`` is in
    descending order): the starting point of the search for the capacity addition; it tends to overshoot."""
    cap = _padded_capacity(base_avg, 0, goal, num_gpus, grad_accum)
    longest = int(sorted_lengths[0])
    n = max(1, min(len(sorted_lengths), cap // max(longest, 1)))
    return round(sum(longest - int(x) for x in sorted_lengths[:n]) / n)


def simulate_buckets(base_avg, goal, num_gpus, grad_accum, pad_id, max_batch_len, lengths, seed, dataset, addition) -> float:
    """Average number of samples per step that padded multipack batches give when the per-GPU capacity is raised by
    ``addition`` tokens per sample.  ``pad_id``, ``max_batch_len`` and ``dataset`` are accepted for the reference's
    calling convention; only the lengths matter."""
    import os as _os

    cap = _padded_capacity(base_avg, addition, goal, num_gpus, grad_accum)
    world = int(_os.environ.get("WORLD_SIZE", num_gpus))
    rank = int(_os.environ.get("RANK", 0))
    sampler = MultipackDistributedBatchSampler(cap, np.asarray(lengths), world, rank, seed, padding=True)
    n_batches = len(sampler.generate_batches())
    return len(lengths) / n_batches if n_batches else 0.0


def find_padding_max_batch_len_addition(base_avg, goal, dataset, num_gpus, grad_accum, pad_id, max_batch_len, seed) -> int:
    """Tokens per sample to add to the unpadded capacity so that padded batches still average ``goal`` samples per
    step (within 2 %, at least 10 samples): bracket from the first-bucket guess, doubling the upper end until the
    simulation overshoots, then bisect."""
    if hasattr(dataset, "get_lengths"):
        lengths = np.asarray(dataset.get_lengths())
    else:  # plain lengths, or samples that carry their tokens
        lengths = np.asarray([len(s["input_ids"]) if isinstance(s, dict) else int(s) for s in dataset])
    guess = guess_starting_avg_padding(base_avg, goal, num_gpus, grad_accum, sorted(lengths.tolist(), reverse=True))
    lo, hi, cur, overshot = 0, max(2 * guess, 2), max(guess, 1), False
    tol = max(10, round(goal * 0.02))
    for _ in range(64):
        if hi - lo <= 1:
            break
        got = simulate_buckets(base_avg, goal, num_gpus, grad_accum, pad_id, max_batch_len, lengths, seed, dataset, cur)
        if abs(got - goal) <= tol:
            break
        if got > goal:
            overshot, hi = True, cur
        elif not overshot:
            hi *= 2
        else:
            lo = cur
        cur = lo + (hi - lo) // 2
    return cur
