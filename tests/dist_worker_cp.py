"""Context-parallel Mamba2 check run under torchrun by tests/dist_worker.py."""
import torch
import torch.distributed as dist


def check_cp(dev, rank, world):
    from fms_acceleration_b200 import _native as NV
    from fms_acceleration_b200.models.builder import build_model
    from fms_acceleration_b200.models.config import DecoderConfig
    from fms_acceleration_b200.parallel.engine import ShardedEngine
    from fms_acceleration_b200.plugins.mcp.utils import patch_mamba_layers_with_cp_head

    cfg = DecoderConfig(vocab_size=512, hidden_size=256, num_hidden_layers=2, num_attention_heads=8,
                        model_type="mamba2", architectures=["Mamba2ForCausalLM"], mamba_d_state=64, mamba_d_head=64,
                        mamba_expand=2, mamba_d_conv=4, mamba_chunk_size=64, rms_norm_eps=1e-5, tie_word_embeddings=True)
    T = 256 * world
    torch.manual_seed(0)
    ids = torch.randint(0, 512, (1, T), device=dev)

    def make():
        m = build_model(cfg, device=dev, dtype=torch.bfloat16, seed=0)
        m.enable_fused("fused_ce_liger")
        return m

    ref = make()
    ref_loss = ref(ids, labels=ids).loss
    ref_loss.backward()
    ref_grads = {n: p.grad.float().clone() for n, p in ref.named_parameters()}

    model = make()
    patch_mamba_layers_with_cp_head(model, None, rank, cp_degree=world, world_size=world)
    engine = ShardedEngine(model, shard_frozen=False, grad_scale=1.0)
    sl = slice(rank * (T // world), (rank + 1) * (T // world))
    for it in range(2):
        engine.zero_grad()
        out = model(ids[:, sl], labels=ids[:, sl])
        out.loss.backward()
        engine.reduce_gradients()
    NV.check_status()
    total = out.loss.detach().float().clone()
    dist.all_reduce(total)
    assert abs(total.item() - ref_loss.item()) < 2e-2 * max(1.0, abs(ref_loss.item())), (total.item(), ref_loss.item())
    worst = 0.0
    for n, p in model.named_parameters():
        r = ref_grads[n]
        if r.norm() < 1e-8:
            continue
        err = ((p.grad.float() - r).norm() / r.norm()).item()
        worst = max(worst, err)
        assert err < 8e-2, (n, err)
    print(f"DIST_OK mamba_cp (loss {total.item():.4f} vs {ref_loss.item():.4f}, worst grad err {worst:.2e})", flush=True)
