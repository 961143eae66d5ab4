"""Multi-rank test body, launched by ``tests/test_gpu_multi.py`` with torchrun (one rank per GPU, NCCL for the
bootstrap, the package's own peer-memory kernels for the data plane).  Prints ``DIST_OK <name>`` per passed check."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def check_comm(dev, rank, world):
    from fms_acceleration_b200 import _native as NV
    from fms_acceleration_b200.parallel.symm import Communicator, SymmBuffer

    comm = Communicator()
    torch.manual_seed(rank)
    # all-gather against NCCL
    shard_bytes = 1 << 20
    shards = SymmBuffer(shard_bytes * 3)
    shards.local.copy_(torch.randint(0, 256, (shards.nbytes,), dtype=torch.uint8, device=dev))
    comm.barrier(0)
    dst = torch.empty(shard_bytes * world, dtype=torch.uint8, device=dev)
    comm.allgather_into(shards, shard_bytes, shard_bytes, dst)
    ref = [torch.empty(shard_bytes, dtype=torch.uint8, device=dev) for _ in range(world)]
    dist.all_gather(ref, shards.local[shard_bytes: 2 * shard_bytes].contiguous())
    assert torch.equal(dst, torch.cat(ref)), "allgather mismatch"
    print("DIST_OK allgather", flush=True)
    # all-reduce (bf16 and fp32) against NCCL
    for dtype in (torch.bfloat16, torch.float32):
        n = world * 16 * 1024 * 3
        esz = torch.empty((), dtype=dtype).element_size()
        bucket = SymmBuffer(n * esz)
        x = torch.randn(n, device=dev).to(dtype)
        bucket.view(0, n, dtype).copy_(x)
        for it in range(3):
            bucket.view(0, n, dtype).copy_(x)
            comm.allreduce_(bucket, n, dtype)
        NV.check_status()
        ref = x.float().clone()
        dist.all_reduce(ref)
        ref = ref / world
        got = bucket.view(0, n, dtype).float()
        tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
        assert torch.allclose(got, ref, rtol=tol, atol=tol), f"allreduce {dtype} mismatch {(got - ref).abs().max()}"
    # the same through the switch's multicast object (in-switch reduction), where the fabric offers one
    n = world * 16 * 1024 * 3
    for dtype in (torch.bfloat16, torch.float32):
        esz = torch.empty((), dtype=dtype).element_size()
        bucket = SymmBuffer(n * esz)
        if not bucket.mc_ptr:
            print("multimem: no multicast object on this fabric, skipped", flush=True)
            break
        x = torch.randn(n, device=dev).to(dtype)
        for it in range(2):
            bucket.view(0, n, dtype).copy_(x)
            comm.barrier(0)
            comm.allreduce_(bucket, n, dtype, multimem=True)
        NV.check_status()
        ref = x.float().clone()
        dist.all_reduce(ref)
        got = bucket.view(0, n, dtype).float()
        tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
        assert torch.allclose(got, ref / world, rtol=tol, atol=tol), f"multimem allreduce {dtype} mismatch"
    else:
        print("multimem allreduce checked against NCCL", flush=True)
    print("DIST_OK allreduce", flush=True)
    # reduce-scatter with fused scale and fp32 output
    n_own = 8 * 4096
    bucket = SymmBuffer(n_own * world * 2)
    x = torch.randn(n_own * world, device=dev).bfloat16()
    bucket.view(0, n_own * world, torch.bfloat16).copy_(x)
    out = torch.empty(n_own, dtype=torch.float32, device=dev)
    comm.reduce_scatter(bucket, n_own, torch.bfloat16, out, scale=0.5)
    NV.check_status()
    full = x.float().clone()
    dist.all_reduce(full)
    assert torch.allclose(out, 0.5 * full[rank * n_own: (rank + 1) * n_own], rtol=1e-5, atol=1e-5)
    print("DIST_OK reduce_scatter", flush=True)


def check_engine(dev, rank, world):
    """Sharded QLoRA training equals the same model trained unsharded on the concatenated batch."""
    from fms_acceleration_b200 import _native as NV
    from fms_acceleration_b200.models.builder import build_model, quantize_linears_
    from fms_acceleration_b200.models.config import DecoderConfig
    from fms_acceleration_b200.nn import Linear4bit, LoraConfig, get_peft_model
    from fms_acceleration_b200.parallel.engine import ShardedEngine
    from fms_acceleration_b200.trainer import TrainArgs, Trainer, synthetic_packed_batch

    cfg = DecoderConfig(vocab_size=2048, hidden_size=512, intermediate_size=1024, num_hidden_layers=3,
                        num_attention_heads=4, num_key_value_heads=2, head_dim=128)

    def make():
        torch.manual_seed(0)
        m = build_model(cfg, device=dev, dtype=torch.bfloat16, layer_hook=lambda l: quantize_linears_(
            l, lambda lin: Linear4bit.from_linear(lin, "nf4", 64, torch.bfloat16)))
        m.quantization_method = "bitsandbytes"
        m = get_peft_model(m, LoraConfig(r=16, lora_alpha=16, target_modules=["q_proj", "k_proj", "v_proj", "o_proj"]))
        torch.manual_seed(1)
        for n, p in m.named_parameters():
            if "lora_B" in n:
                torch.nn.init.normal_(p, std=0.02)
        m.get_base_model().enable_fused("fused_ce_liger")
        return m

    batches = [synthetic_packed_batch(2048, 1, 512, (32, 512), seed=100 + r, pin=False) for r in range(world)]
    # reference: every rank computes the average of the per-rank gradients on an unsharded replica
    ref = make()
    ref_grads = None
    for b in batches:
        out = ref(**{k: v.to(dev) for k, v in b.items() if k != "cu_seqlens"})
        out.loss.backward()
    ref_grads = {n: p.grad.float() / world for n, p in ref.named_parameters() if p.grad is not None}

    model = make()
    engine = ShardedEngine(model)
    assert engine.arena is not None and len(engine.blobs) == 3
    b = batches[rank]
    out = model(**{k: v.to(dev) for k, v in b.items() if k != "cu_seqlens"})
    out.loss.backward()
    engine.reduce_gradients()
    NV.check_status()
    worst = 0.0
    for n, p in model.named_parameters():
        if p.grad is None:
            continue
        r = ref_grads[n]
        if r.norm() < 1e-8:
            continue
        err = ((p.grad.float() - r).norm() / r.norm()).item()
        worst = max(worst, err)
    assert worst < 3e-2, f"sharded vs replicated gradient mismatch {worst}"
    print(f"DIST_OK engine (worst rel grad err {worst:.2e})", flush=True)
    # a few optimizer steps run and the loss moves
    tr = Trainer(model, TrainArgs(bf16=True, learning_rate=1e-3), engine=engine)
    engine.zero_grad()
    l0 = float(tr.train_step(b))
    for _ in range(3):
        l1 = float(tr.train_step(b))
    NV.check_status()
    assert l1 < l0, (l0, l1)
    print("DIST_OK engine_train", flush=True)


def check_zero1(dev, rank, world):
    """Optimizer-state sharding: a full fine-tune in fp32 with the sharded AdamW ends at the same parameters as the
    replicated optimizer (all-reduced gradients), and every rank holds the same parameters afterwards."""
    from fms_acceleration_b200 import _native as NV
    from fms_acceleration_b200.models.builder import build_model
    from fms_acceleration_b200.models.config import DecoderConfig
    from fms_acceleration_b200.parallel.engine import ShardedEngine
    from fms_acceleration_b200.trainer import TrainArgs, Trainer, synthetic_packed_batch

    cfg = DecoderConfig(vocab_size=512, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                        num_attention_heads=4, num_key_value_heads=2, head_dim=64)
    batches = [synthetic_packed_batch(512, 1, 256, (32, 256), seed=7 * rank + i, pin=False) for i in range(3)]

    def run(shard: bool):
        torch.manual_seed(0)
        m = build_model(cfg, device=dev, dtype=torch.float32, seed=0)
        eng = ShardedEngine(m, shard_frozen=False, shard_optimizer=shard)
        tr = Trainer(m, TrainArgs(learning_rate=1e-3, weight_decay=0.01, max_grad_norm=1.0), engine=eng)
        assert (tr.optimizer is eng.sharded_optimizer) == shard
        eng.zero_grad()
        losses = [float(tr.train_step(b)) for b in batches]
        NV.check_status()
        return m, losses, tr

    m_ref, l_ref, _ = run(False)
    m_sh, l_sh, tr = run(True)
    assert abs(l_ref[0] - l_sh[0]) < 1e-5
    worst = 0.0
    for (n, a), (_, b) in zip(m_ref.named_parameters(), m_sh.named_parameters()):
        worst = max(worst, ((a - b).norm() / a.norm().clamp(min=1e-9)).item())
    assert worst < 2e-4, worst
    flat = m_sh.lm_head.weight.detach().clone()
    other = flat.clone()
    dist.broadcast(other, src=0)
    assert torch.equal(flat, other)  # every rank pulled the same updated slices
    n_state = sum(v.numel() for st in tr.optimizer.inner.state.values() for v in st.values() if torch.is_tensor(v))
    n_params = sum(p.numel() for p in m_sh.parameters())
    assert n_state <= 2 * (n_params // world + 4096) + 8  # two moments over 1/world of the parameters
    print(f"DIST_OK zero1 (worst rel parameter diff {worst:.1e}, state elements {n_state})", flush=True)


def main():
    rank = int(os.environ["RANK"])
    world = int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    which = sys.argv[1] if len(sys.argv) > 1 else "all"
    if which in ("all", "comm"):
        check_comm(dev, rank, world)
    if which in ("all", "engine"):
        check_engine(dev, rank, world)
    if which in ("all", "zero1"):
        check_zero1(dev, rank, world)
    if which in ("all", "moe") and os.path.exists(os.path.join(os.path.dirname(__file__), "dist_worker_moe.py")):
        from dist_worker_moe import check_moe, check_moe_library, check_moe_lora

        check_moe(dev, rank, world)
        check_moe_library(dev, rank, world)
        check_moe_lora(dev, rank, world)
    if which in ("all", "cp"):
        from dist_worker_cp import check_cp

        check_cp(dev, rank, world)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
