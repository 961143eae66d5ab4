"""Worker of test_engine_cpu: the host-side logic of the sharded engine, the rank-sharded optimizer, gradient
accumulation and the expert-parallel checkpoint on gloo ranks (CPU tensors, library collectives in place of the
peer-memory kernels)."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def _batches(vocab, rank, n, seq=48, seed=0):
    from fms_acceleration_b200.trainer import synthetic_packed_batch

    return [synthetic_packed_batch(vocab, 2, seq, (8, seq), seed=seed + 100 * rank + i, pin=False) for i in range(n)]


def check_overlapped_reduce(rank, world):
    """Segments reduced from the autograd hooks equal the plain mean of the per-rank gradients; two micro-batches
    with accumulation equal one step on their mean gradient."""
    from fms_acceleration_b200.models.builder import build_model
    from fms_acceleration_b200.parallel.engine import ShardedEngine

    os.environ["FMSB_GRAD_SEGMENT_MB"] = "0.05"  # several segments even for the tiny model
    torch.manual_seed(0)
    model = build_model("tiny-llama", dtype=torch.float32, seed=0)
    eng = ShardedEngine(model, shard_frozen=False, backend="library")
    assert len(eng.segments) > 2, len(eng.segments)
    b = _batches(model.config.vocab_size, rank, 2)
    eng.zero_grad()
    eng.begin_micro_step(True)
    model(**b[0]).loss.backward()
    assert all(s.launched for s in eng.segments)  # every segment was reduced from its hook, during backward
    eng.reduce_gradients()
    got = {n: p.grad.clone() for n, p in model.named_parameters()}
    ref = build_model("tiny-llama", dtype=torch.float32, seed=0)
    ref(**b[0]).loss.backward()
    for n, p in ref.named_parameters():
        g = p.grad.clone()
        dist.all_reduce(g)
        assert torch.allclose(got[n], g / world, atol=1e-6), n
    # accumulation: nothing is reduced before the last micro-batch
    eng.zero_grad()
    eng.begin_micro_step(False)
    (model(**b[0]).loss / 2).backward()
    eng.end_micro_step()
    assert not any(s.launched for s in eng.segments)
    eng.begin_micro_step(True)
    (model(**b[1]).loss / 2).backward()
    eng.end_micro_step()
    eng.reduce_gradients()
    ref.zero_grad()
    (ref(**b[0]).loss / 2).backward()
    (ref(**b[1]).loss / 2).backward()
    for n, p in ref.named_parameters():
        g = p.grad.clone()
        dist.all_reduce(g)
        assert torch.allclose(dict(model.named_parameters())[n].grad, g / world, atol=1e-6), n
    print("CPU_OK overlapped_reduce", flush=True)


def check_zero1_and_resume(rank, world, tmp):
    """The rank-sharded AdamW ends at the same parameters as the replicated one; its state goes through one
    distributed-checkpoint directory and a resumed run continues bit for bit."""
    from fms_acceleration_b200.models.builder import build_model
    from fms_acceleration_b200.parallel.engine import ShardedEngine
    from fms_acceleration_b200.trainer import TrainArgs, Trainer

    os.environ["FMSB_GRAD_SEGMENT_MB"] = "0.05"

    def make(shard, out):
        torch.manual_seed(0)
        m = build_model("tiny-llama", dtype=torch.float32, seed=0)
        eng = ShardedEngine(m, shard_frozen=False, shard_optimizer=shard, backend="library")
        tr = Trainer(m, TrainArgs(learning_rate=1e-3, weight_decay=0.01, max_grad_norm=1.0, output_dir=out), engine=eng)
        assert (tr.optimizer is eng.sharded_optimizer) == shard
        eng.zero_grad()
        return m, tr

    V = 1024
    bs = _batches(V, rank, 5)
    m_ref, tr_ref = make(False, os.path.join(tmp, "ref"))
    l_ref = [float(tr_ref.train_step(b)) for b in bs]
    m_sh, tr_sh = make(True, os.path.join(tmp, "sh"))
    l_a = [float(tr_sh.train_step(b)) for b in bs[:3]]
    ckpt = tr_sh.save_checkpoint()
    l_a += [float(tr_sh.train_step(b)) for b in bs[3:]]
    assert max(abs(a - b) for a, b in zip(l_ref, l_a)) < 1e-4, (l_ref, l_a)
    for (n, a), (_, b) in zip(m_ref.named_parameters(), m_sh.named_parameters()):
        # AdamW divides by sqrt(v) + eps: where a gradient element is itself of the order of eps (a few entries of the
        # embedding), rounding-level differences between the two runs are amplified to a fraction of one update.
        # Everything else agrees to rounding.
        d = (a - b).abs()
        assert ((a - b).norm() / a.norm()).item() < 1e-5, n
        assert (d > 2e-6).float().mean().item() < 1e-4, n
    # every rank holds the same parameters
    flat = tr_sh.engine.flat_params.clone()
    other = flat.clone()
    dist.broadcast(other, src=0)
    assert torch.equal(flat, other)
    # resume from step 3 in a fresh process state
    m_re, tr_re = make(True, os.path.join(tmp, "re"))
    tr_re.load_checkpoint(ckpt)
    assert tr_re.global_step == 3
    l_b = [float(tr_re.train_step(b)) for b in bs[3:]]
    assert l_b == l_a[3:], (l_b, l_a[3:])
    for (n, a), (_, b) in zip(m_sh.named_parameters(), m_re.named_parameters()):
        assert torch.equal(a, b), n
    # nothing but distributed-checkpoint directories: no per-rank side files
    assert not [f for f in os.listdir(ckpt) if f.startswith("optimizer_shard")]
    print("CPU_OK zero1_resume", flush=True)


def check_ep_checkpoint(rank, world, tmp):
    """Expert parallelism over all ranks: two training steps, save, convert to safetensors without a process group:
    every rank's experts are in the file, equal to the gathered shards bit for bit; a fresh model resumes exactly."""
    from safetensors.torch import load_file, save_file

    from fms_acceleration_b200.models.builder import build_model
    from fms_acceleration_b200.parallel.engine import ShardedEngine
    from fms_acceleration_b200.plugins.moe.utils import checkpoint_utils as CU
    from fms_acceleration_b200.plugins.moe.utils import prepare_scattermoe
    from fms_acceleration_b200.trainer import TrainArgs, Trainer

    pretrained = os.path.join(tmp, "pretrained")
    torch.manual_seed(0)
    base = build_model("tiny-granitemoe", dtype=torch.float32, seed=0)
    original = {k: v.clone().contiguous() for k, v in base.state_dict().items() if k != "lm_head.weight"}
    if rank == 0:
        os.makedirs(pretrained, exist_ok=True)
        save_file(original, os.path.join(pretrained, "model.safetensors"), metadata={"format": "pt"})
        with open(os.path.join(pretrained, "config.json"), "w") as fh:
            json.dump({"architectures": ["GraniteMoeForCausalLM"]}, fh)
    dist.barrier()

    def make(seed, out):
        m = build_model("tiny-granitemoe", dtype=torch.float32, seed=seed)
        prepare_scattermoe(m, None, rank, world, world)
        eng = ShardedEngine(m, shard_frozen=False, backend="library")
        assert eng.ep_params and eng.params
        tr = Trainer(m, TrainArgs(learning_rate=1e-2, max_grad_norm=1.0, output_dir=out), engine=eng)
        eng.zero_grad()
        return m, tr

    bs = _batches(1024, rank, 4, seq=32)
    m, tr = make(0, os.path.join(tmp, "ep"))
    la = [float(tr.train_step(b)) for b in bs[:2]]
    ckpt = tr.save_checkpoint()
    la += [float(tr.train_step(b)) for b in bs[2:]]
    # replicated parameters stayed identical across the ranks although the expert gradients differ per rank
    w = m.model.layers[0].self_attn.q_proj.weight.detach().clone()
    w0 = w.clone()
    dist.broadcast(w0, src=0)
    assert torch.equal(w, w0)
    # resume
    m2, tr2 = make(1, os.path.join(tmp, "ep2"))
    tr2.load_checkpoint(ckpt)
    lb = [float(tr2.train_step(b)) for b in bs[2:]]
    assert lb == la[2:], (lb, la[2:])
    # conversion without a process group, on rank 0, from the step-2 checkpoint
    m3, tr3 = make(2, os.path.join(tmp, "ep3"))
    tr3.load_checkpoint(ckpt)
    sd = {k: v.detach().clone() for k, v in m3.state_dict().items()}
    gathered = {}
    for k, v in sd.items():
        if any(f".{wn}.weight" in k for wn in ("w1", "w2", "w3")):
            parts = [torch.empty_like(v) for _ in range(world)]
            dist.all_gather(parts, v.contiguous())
            gathered[k] = torch.cat(parts, 0)
        else:
            gathered[k] = v
    if rank == 0:
        out = os.path.join(tmp, "hf")
        CU.recover_safetensors_from_dcp(ckpt, pretrained, out)
        rec = load_file(os.path.join(out, "model.safetensors"))
        want = CU.recover_original_state_dict_from_checkpoint(dict(gathered), weight_map={k: "x" for k in original},
                                                              architectures=["GraniteMoeForCausalLM"])
        for k in original:
            assert k in rec and rec[k].shape == original[k].shape, k
            assert torch.equal(rec[k], want[k]), k
        moved = sum(int(not torch.equal(rec[k], original[k])) for k in original)
        assert moved > len(original) // 2  # the checkpoint holds trained weights, not the initial ones
    dist.barrier()
    print("CPU_OK ep_checkpoint", flush=True)


def check_ep_lora(rank, world, tmp):
    """Per-expert LoRA under expert parallelism (adapters are created per local expert, base experts frozen): the
    plugin accepts it, only adapters and nothing else of the experts trains, the loss goes down, and the adapter
    checkpoint holds every rank's adapters."""
    from fms_acceleration_b200.models.builder import build_model
    from fms_acceleration_b200.nn.lora import LoraConfig
    from fms_acceleration_b200.parallel.engine import ShardedEngine
    from fms_acceleration_b200.plugins.moe.framework_plugin_scattermoe import ScatterMoEAccelerationPlugin
    from fms_acceleration_b200.plugins.moe.utils import checkpoint_utils as CU
    from fms_acceleration_b200.trainer import TrainArgs, Trainer

    model = build_model("tiny-granitemoe", dtype=torch.float32, seed=0)
    plugin = ScatterMoEAccelerationPlugin({"training": {"moe": {"scattermoe": {"ep_degree": world}}}})
    targs = TrainArgs(learning_rate=5e-2, output_dir=os.path.join(tmp, "lora"))
    cfg = LoraConfig(r=4, lora_alpha=8, target_modules=["all-linear"])
    model, _ = plugin.augmentation(model, targs, modifiable_args=(cfg,))
    for n, p in model.named_parameters():  # a LoRA run trains adapters only
        p.requires_grad_("lora_" in n)
    moe = model.model.layers[0].block_sparse_moe
    assert moe.w1.lora_A.shape[0] == moe.num_experts // world and not moe.w1.weight.requires_grad
    eng = ShardedEngine(model, shard_frozen=False, backend="library")
    assert eng.ep_params and all("lora" in n for n, p in model.named_parameters() if p.requires_grad)
    tr = Trainer(model, targs, engine=eng)
    eng.zero_grad()
    b = _batches(1024, rank, 1, seq=32)[0]
    w0 = moe.w1.weight.detach().clone()
    losses = [float(tr.train_step(b)) for _ in range(6)]
    assert losses[-1] < losses[0], losses
    assert torch.equal(moe.w1.weight, w0)
    ckpt = tr.save_checkpoint()
    dist.barrier()
    if rank == 0:
        sd = CU.get_state_dict_from_dcp_checkpoint(os.path.join(ckpt, "pytorch_model_fsdp_0"))
        key = [k for k in sd if k.endswith("layers.0.block_sparse_moe.w1.lora_A")][0]
        assert sd[key].shape[0] == moe.num_experts  # all ranks' adapters, not one rank's
    dist.barrier()
    print("CPU_OK ep_lora", flush=True)


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    which, tmp = sys.argv[1], sys.argv[2]
    if which == "reduce":
        check_overlapped_reduce(rank, world)
    elif which == "zero1":
        check_zero1_and_resume(rank, world, tmp)
    elif which == "ep_ckpt":
        check_ep_checkpoint(rank, world, tmp)
    elif which == "ep_lora":
        check_ep_lora(rank, world, tmp)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
