"""Worker of test_cp_baseline_cpu: causal attention of one sequence split over gloo ranks (keys / values gathered over
the group) equals the attention of the whole sequence, outputs and gradients; then the same through a hybrid
decoder layer whose attention block runs context-parallel."""
import os
import sys

import torch
import torch.distributed as dist
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    from fms_acceleration_b200.parallel.context_parallel import cp_attention

    torch.manual_seed(0)  # the same full sequence on every rank
    Tl, nh, nkv, d = 40, 4, 2, 16
    T = Tl * world
    q = torch.randn(T, nh, d, dtype=torch.float64, requires_grad=True)
    k = torch.randn(T, nkv, d, dtype=torch.float64, requires_grad=True)
    v = torch.randn(T, nkv, d, dtype=torch.float64, requires_grad=True)
    g = torch.randn(T, nh, d, dtype=torch.float64)
    scale = 0.3
    rep = nh // nkv
    full = F.scaled_dot_product_attention(q.transpose(0, 1)[None], k.repeat_interleave(rep, 1).transpose(0, 1)[None],
                                          v.repeat_interleave(rep, 1).transpose(0, 1)[None], is_causal=True, scale=scale)
    full = full[0].transpose(0, 1)
    (full * g).sum().backward()
    sl = slice(rank * Tl, (rank + 1) * Tl)
    ql, kl, vl = (t.detach()[sl].clone().requires_grad_() for t in (q, k, v))
    out = cp_attention(ql, kl, vl, dist.group.WORLD, scale, q_block=16)
    assert torch.allclose(out, full[sl].detach(), atol=1e-10), (out - full[sl]).abs().max()
    (out * g[sl]).sum().backward()
    assert torch.allclose(ql.grad, q.grad[sl], atol=1e-10)
    assert torch.allclose(kl.grad, k.grad[sl], atol=1e-10), (kl.grad - k.grad[sl]).abs().max()
    assert torch.allclose(vl.grad, v.grad[sl], atol=1e-10)

    # a hybrid decoder layer with an attention block: the context-parallel layer on a slice against the plain layer
    from types import SimpleNamespace

    from fms_acceleration_b200.models.builder import resolve_config
    from fms_acceleration_b200.models.granitemoehybrid import GraniteMoeHybridDecoderLayer

    cfg = resolve_config("tiny-granitemoehybrid")
    idx = [i for i, t in enumerate(cfg.layer_types) if t != "mamba"][0]
    torch.manual_seed(1)
    layer = GraniteMoeHybridDecoderLayer(cfg, idx).double()
    x = torch.randn(T, cfg.hidden_size, dtype=torch.float64)
    pos = torch.zeros(T, dtype=torch.long)
    cos_t, sin_t = torch.ones(1, cfg.head_dim // 2, dtype=torch.float64), torch.zeros(1, cfg.head_dim // 2, dtype=torch.float64)
    with torch.no_grad():
        ref = layer(x, pos, cos_t, sin_t, [0, T])
        layer.cp = SimpleNamespace(group=dist.group.WORLD)
        mine = layer(x[sl], pos[sl], cos_t, sin_t, [0, Tl])
    assert torch.allclose(mine, ref[sl], atol=1e-8), (mine - ref[sl]).abs().max()
    dist.barrier()
    if rank == 0:
        print("CP_ATTENTION_OK")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
