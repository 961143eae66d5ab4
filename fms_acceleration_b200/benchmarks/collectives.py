"""Communication kernels in isolation, beside the NCCL collective that does the same job.

Launch with one process per GPU::

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29655 \
        -m fms_acceleration_b200.benchmarks.collectives [--sizes-mb 54 1024] [--iters 20] [--multimem]

Every line is timed with CUDA events on the launching stream after warm-up, a barrier and a device synchronisation on
both sides, and is the MAX over the ranks.  Reported per size:

* ``allreduce_p2p``: the one-kernel two-shot all-reduce of a flat fp32 bucket (``csrc/comm.cu``), the gradient
  reduction of adapter runs;
* ``allreduce_multimem`` (``--multimem``): the same through the NVSwitch multicast object;
* ``reduce_scatter`` and ``all_gather``: the ZeRO-1 pair of a full fine-tune (bf16 buckets, fp32 gradient slice);
* the NCCL forms of each (``dist.all_reduce``, ``reduce_scatter_tensor``, ``all_gather_into_tensor``).

Bus bandwidth follows the usual convention: all-reduce ``2 (N-1)/N * bytes / t``, reduce-scatter and all-gather
``(N-1)/N * bytes / t``; the peer-copy figure measured on this kind of machine is 770 GB/s per direction and GPU.
The reference runs these collectives through NCCL under FSDP / DDP (scripts/benchmarks/accelerate.yaml).
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def _timed(fn, iters: int, warmup: int) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    t = torch.tensor([s.elapsed_time(e) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--sizes-mb", type=float, nargs="+", default=[54.0, 1024.0])
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--multimem", action="store_true", help="also time the NVSwitch multicast all-reduce")
    ap.add_argument("--ag-ctas", type=int, default=96, help="CTAs of the all-gather pull (the engine uses 96 after the step)")
    a = ap.parse_args()

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    from fms_acceleration_b200 import _native as NV
    from fms_acceleration_b200.parallel.symm import Communicator, SymmBuffer

    dev = torch.device("cuda", torch.cuda.current_device())
    comm = Communicator(device=dev)
    out = []

    def report(rec):
        if rank == 0:
            print(json.dumps(rec), flush=True)
        out.append(rec)

    for mb in a.sizes_mb:
        n32 = int(mb * (1 << 20)) // 4 // (world * 64) * (world * 64)
        nbytes = n32 * 4
        bucket = SymmBuffer(nbytes, device=dev)
        flat = bucket.view(0, n32, torch.float32)
        flat.fill_(1.0)
        ar = 2.0 * (world - 1) / world * nbytes
        t = _timed(lambda: comm.allreduce_(bucket, n32, torch.float32, scale=1.0 / world, multimem=False), a.iters, a.warmup)
        NV.check_status()
        ok = bool(torch.allclose(flat[:1024], torch.ones(1024, device=dev)))
        report({"op": "allreduce_p2p fp32", "mb": mb, "ms": t, "busbw_gbs": ar / t / 1e6, "n_gpus": world, "result_ok": ok})
        if a.multimem and bucket.mc_ptr:
            flat.fill_(1.0)
            t = _timed(lambda: comm.allreduce_(bucket, n32, torch.float32, scale=1.0 / world, multimem=True), a.iters, a.warmup)
            NV.check_status()
            ok = bool(torch.allclose(flat[:1024], torch.ones(1024, device=dev)))
            report({"op": "allreduce_multimem fp32", "mb": mb, "ms": t, "busbw_gbs": ar / t / 1e6, "n_gpus": world,
                    "result_ok": ok})
        ref = torch.ones(n32, device=dev)
        t = _timed(lambda: dist.all_reduce(ref), a.iters, a.warmup)
        report({"op": "nccl all_reduce fp32", "mb": mb, "ms": t, "busbw_gbs": ar / t / 1e6, "n_gpus": world})
        del ref
        # ZeRO-1 pair on the same bytes viewed as bf16: reduce-scatter to an fp32 slice, all-gather of the bf16 slices
        n16 = nbytes // 2
        own = n16 // world
        gslice = torch.empty(own, dtype=torch.float32, device=dev)
        half = (world - 1) / world * nbytes

        full16 = bucket.view(0, n16, torch.bfloat16)
        full16.fill_(1.0)

        def rs():
            comm.reduce_scatter(bucket, own, torch.bfloat16, gslice, scale=1.0 / world)

        def ag():
            # every rank pulls slice r from rank r's bucket into its own copy (the parameter all-gather of the engine)
            comm.barrier(6)
            rc = NV.lib().fmsb_comm_allgather(bucket.ptr_array_strided(0, own * 2), full16.data_ptr(), own * 2, rank,
                                              world, a.ag_ctas, NV.stream_ptr())
            NV.check(rc, "fmsb_comm_allgather")
            comm.barrier(7)

        t_rs = _timed(rs, a.iters, a.warmup)
        NV.check_status()
        t_ag = _timed(ag, a.iters, a.warmup)
        NV.check_status()
        report({"op": "reduce_scatter bf16 -> fp32 slice (p2p kernel, 64 CTAs, barriers included)", "mb": mb, "ms": t_rs,
                "busbw_gbs": half / t_rs / 1e6, "n_gpus": world})
        report({"op": "all_gather bf16 (p2p kernel, %d CTAs, barriers included)" % a.ag_ctas, "mb": mb, "ms": t_ag,
                "busbw_gbs": half / t_ag / 1e6, "n_gpus": world})
        src = torch.ones(n16, dtype=torch.bfloat16, device=dev)
        dst = torch.empty(own, dtype=torch.bfloat16, device=dev)

        t_rs = _timed(lambda: dist.reduce_scatter_tensor(dst, src), a.iters, a.warmup)
        t_ag = _timed(lambda: dist.all_gather_into_tensor(src, dst), a.iters, a.warmup)
        report({"op": "nccl reduce_scatter_tensor bf16", "mb": mb, "ms": t_rs, "busbw_gbs": half / t_rs / 1e6, "n_gpus": world})
        report({"op": "nccl all_gather_into_tensor bf16", "mb": mb, "ms": t_ag, "busbw_gbs": half / t_ag / 1e6, "n_gpus": world})
        del src, dst, gslice, flat, full16, bucket
        torch.cuda.empty_cache()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
