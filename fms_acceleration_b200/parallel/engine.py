"""Sharded-parameter engine (the role accelerate's FSDP plays for the reference).

* **Frozen quantised base weights** (QLoRA / GPTQ-LoRA): every decoder layer's packed tensors are flattened into
  one byte blob; each rank keeps 1/world of it in a symmetric arena and the full copies are freed.  A layer is
  materialised right before it runs by pulling the peers' slices over NVLink into one of two staging buffers
  (``csrc/comm.cu``), prefetched one layer ahead on a side stream, in forward and again (in reverse order) in
  backward.  The weights never change, so the ranks need no synchronisation for this at all.
* **Trainable replicated parameters** (LoRA adapters, or everything in full fine-tuning): their gradients live
  as views inside one flat symmetric bucket; after backward ONE kernel averages the bucket across ranks
  (two-shot all-reduce over peer memory with the 1/world scale and the cast fused in).  With
  ``shard_optimizer=True`` the bucket is reduce-scattered instead, each rank steps its slice of an fp32 master
  copy and the updated parameters are all-gathered (ZeRO-1).

The reference reaches the same ends with accelerate FSDP plus 256 per-tensor NCCL all-reduce hooks for the
adapters (fms_acceleration_foak/utils.py:27-80).
"""
from __future__ import annotations

import os

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist
from torch import nn

from .symm import Communicator, SymmBuffer

_SHARDABLE_BUFFERS = {
    "Linear4bit": ("weight", "absmax_q", "absmax2"),
    "QuantLinear": ("qweight", "qzeros", "scales"),
}


def _align(n: int, a: int) -> int:
    return (n + a - 1) // a * a


class _LayerBlob:
    """Byte layout of one layer's quantised tensors inside the (gathered) blob."""

    def __init__(self, layer: nn.Module, world: int):
        self.entries: List[Tuple[nn.Module, str, int, torch.Size, torch.dtype]] = []
        off = 0
        for mod in layer.modules():
            names = _SHARDABLE_BUFFERS.get(mod.__class__.__name__)
            if not names:
                continue
            for n in names:
                t = getattr(mod, n)
                self.entries.append((mod, n, off, t.shape, t.dtype))
                off = _align(off + t.numel() * t.element_size(), 256)
        self.nbytes = _align(off, world * 256)
        self.shard_bytes = self.nbytes // world

    def pack(self, device) -> torch.Tensor:
        blob = torch.zeros(self.nbytes, dtype=torch.uint8, device=device)
        for mod, n, off, shape, dtype in self.entries:
            t = getattr(mod, n).contiguous()
            nb = t.numel() * t.element_size()
            blob[off: off + nb] = t.view(torch.uint8).reshape(-1)
        return blob

    def bind(self, staging: torch.Tensor) -> None:
        """Point the modules' buffers at the gathered bytes."""
        for mod, n, off, shape, dtype in self.entries:
            nb = shape.numel() * torch.empty((), dtype=dtype).element_size()
            mod._buffers[n] = staging[off: off + nb].view(dtype).view(shape)

    def unbind(self) -> None:
        for mod, n, off, shape, dtype in self.entries:
            mod._buffers[n] = torch.empty(0, dtype=dtype, device=mod._buffers[n].device)


class _BackwardTrigger(torch.autograd.Function):
    """Identity in forward; in backward (which runs BEFORE the wrapped layer's backward) calls ``fn``."""

    @staticmethod
    def forward(ctx, x, fn):
        ctx.fn = fn
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        ctx.fn()
        return g, None


class ShardedEngine:
    def __init__(self, model: nn.Module, group: Optional[dist.ProcessGroup] = None, shard_frozen: bool = True,
                 shard_optimizer: bool = False, grad_dtype: Optional[torch.dtype] = None,
                 grad_scale: Optional[float] = None):
        self.model = model
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.device = next(model.parameters()).device
        self.comm = Communicator(self.group, self.device)
        self.comm_stream = torch.cuda.Stream(self.device)
        self.shard_optimizer = shard_optimizer
        self.grad_scale = grad_scale  # None: average (1/world); 1.0: plain sum (context parallelism)
        self.layers = self._find_layers(model)
        self.blobs: List[_LayerBlob] = []
        self.arena: Optional[SymmBuffer] = None
        self.staging: List[torch.Tensor] = []
        self._staged: List[Optional[int]] = [None, None]
        self._ready: List[Optional[torch.cuda.Event]] = [None, None]
        self._released: List[Optional[torch.cuda.Event]] = [None, None]
        if shard_frozen and self.world > 1 and self.layers:
            self._shard_frozen_layers()
        self._setup_grad_bucket(grad_dtype)
        self.sharded_optimizer: Optional["ShardedOptimizer"] = None
        if shard_optimizer and self.world > 1 and self.params:
            self._setup_param_bucket()

    # ------------------------------------------------------------------ frozen quantised weights
    @staticmethod
    def _find_layers(model: nn.Module) -> List[nn.Module]:
        base = model.get_base_model() if hasattr(model, "get_base_model") else model
        inner = getattr(base, "model", None)
        layers = getattr(inner, "layers", None)
        if layers is None:
            return []
        return [l for l in layers if any(m.__class__.__name__ in _SHARDABLE_BUFFERS for m in l.modules())]

    def _shard_frozen_layers(self) -> None:
        self.blobs = [_LayerBlob(l, self.world) for l in self.layers]
        shard_sizes = [b.shard_bytes for b in self.blobs]
        self.shard_offsets = [0]
        for s in shard_sizes:
            self.shard_offsets.append(self.shard_offsets[-1] + s)
        self.arena = SymmBuffer(self.shard_offsets[-1], self.group, self.device, zero=False)
        for i, (layer, blob) in enumerate(zip(self.layers, self.blobs)):
            full = blob.pack(self.device)
            lo = self.rank * blob.shard_bytes
            self.arena.local[self.shard_offsets[i]: self.shard_offsets[i + 1]] = full[lo: lo + blob.shard_bytes]
            blob.unbind()
            del full
        max_bytes = max(b.nbytes for b in self.blobs)
        self.staging = [torch.empty(max_bytes, dtype=torch.uint8, device=self.device) for _ in range(2)]
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)
        torch.cuda.empty_cache()
        for i, layer in enumerate(self.layers):
            self._wrap_layer(i, layer)

    def _issue_gather(self, i: int) -> None:
        """Enqueue the pull of layer ``i`` into its staging slot on the communication stream."""
        if i < 0 or i >= len(self.layers):
            return
        slot = i % 2
        if self._staged[slot] == i:
            return
        cur = torch.cuda.current_stream(self.device)
        with torch.cuda.stream(self.comm_stream):
            if self._released[slot] is not None:
                self.comm_stream.wait_event(self._released[slot])
            blob = self.blobs[i]
            self.comm.allgather_into(self.arena, self.shard_offsets[i], blob.shard_bytes, self.staging[slot], ctas=32)
            ev = torch.cuda.Event()
            ev.record(self.comm_stream)
        self._ready[slot] = ev
        self._staged[slot] = i
        del cur

    def _acquire(self, i: int, prefetch: int) -> None:
        slot = i % 2
        self._issue_gather(i)
        torch.cuda.current_stream(self.device).wait_event(self._ready[slot])
        self.blobs[i].bind(self.staging[slot])
        # the other slot may be refilled once everything enqueued so far on the compute stream is done
        other = 1 - slot
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(self.device))
        self._released[other] = ev
        self._issue_gather(prefetch)

    def _wrap_layer(self, i: int, layer: nn.Module) -> None:
        engine = self
        for attr in ("forward_fused", "forward"):
            orig = getattr(layer, attr)

            def wrapped(x, *args, _orig=orig, _i=i, **kwargs):
                engine._acquire(_i, _i + 1)
                out = _orig(x, *args, **kwargs)
                if torch.is_grad_enabled() and isinstance(out, torch.Tensor) and out.requires_grad:
                    out = _BackwardTrigger.apply(out, lambda: engine._acquire(_i, _i - 1))
                return out

            setattr(layer, attr, wrapped)

    # ------------------------------------------------------------------ gradients of replicated parameters
    def _setup_grad_bucket(self, grad_dtype: Optional[torch.dtype]) -> None:
        # expert-parallel parameters are not replicated over the whole world: they are reduced separately
        self.ep_params = [p for p in self.model.parameters() if p.requires_grad and getattr(p, "_fmsb_expert_parallel", False)]
        self.params = [p for p in self.model.parameters()
                       if p.requires_grad and not getattr(p, "_fmsb_expert_parallel", False)]
        self.bucket = None
        if not self.params:
            return
        dtype = grad_dtype or self.params[0].dtype
        self.grad_dtype = dtype
        esize = torch.empty((), dtype=dtype).element_size()
        n = sum(p.numel() for p in self.params)
        unit = self.world * 16 // esize * 8
        self.bucket_numel = _align(n, unit)
        if self.world > 1:
            self.bucket = SymmBuffer(self.bucket_numel * esize, self.group, self.device)
            flat = self.bucket.view(0, self.bucket_numel, dtype)
        else:
            flat = torch.zeros(self.bucket_numel, dtype=dtype, device=self.device)
        self.flat_grads = flat
        off = 0
        self._grad_views = []
        for p in self.params:
            v = flat[off: off + p.numel()].view_as(p)
            off += p.numel()
            self._grad_views.append(v)
            if p.dtype == dtype:
                p.grad = v
        if self.world > 1:
            # replicated parameters must start identical
            for p in self.params:
                dist.broadcast(p.data, src=dist.get_global_rank(self.group, 0), group=self.group)

    # ------------------------------------------------------------------ optimizer state sharding (ZeRO-1)
    def _setup_param_bucket(self) -> None:
        """Replicated trainable parameters become views into one flat symmetric buffer, laid out like the gradient
        bucket, so that rank r can update slice r and everybody can pull the updated slices."""
        dtypes = {p.dtype for p in self.params}
        if len(dtypes) != 1:
            raise ValueError("optimizer sharding needs all replicated trainable parameters in one dtype")
        self.param_dtype = dtypes.pop()
        esize = torch.empty((), dtype=self.param_dtype).element_size()
        self.param_bucket = SymmBuffer(self.bucket_numel * esize, self.group, self.device)
        flat = self.param_bucket.view(0, self.bucket_numel, self.param_dtype)
        off = 0
        with torch.no_grad():
            for p in self.params:
                v = flat[off: off + p.numel()].view_as(p)
                v.copy_(p.data)
                p.data = v
                off += p.numel()
        self.flat_params = flat
        self.n_own = self.bucket_numel // self.world
        self.own_slice = slice(self.rank * self.n_own, (self.rank + 1) * self.n_own)
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)

    def build_optimizer(self, lr: float, weight_decay: float = 0.0, betas=(0.9, 0.999), eps: float = 1e-8):
        """AdamW over this rank's 1/world slice of the flat parameters (fp32 master copy and moments)."""
        if not hasattr(self, "flat_params"):
            raise RuntimeError("the engine was created without shard_optimizer=True (or runs on one rank)")
        self.sharded_optimizer = ShardedOptimizer(self, lr, weight_decay, betas, eps)
        return self.sharded_optimizer

    def zero_grad(self) -> None:
        for p in self.ep_params:
            p.grad = None
        if not self.params:
            return
        self.flat_grads.zero_()
        for p, v in zip(self.params, self._grad_views):
            if p.dtype == self.grad_dtype:
                p.grad = v
            else:
                p.grad = None

    def _collect_grads(self) -> None:
        """Gradients that autograd did not write straight into the bucket views are copied there."""
        for p, v in zip(self.params, self._grad_views):
            if p.grad is not None and p.grad.data_ptr() != v.data_ptr():
                v.copy_(p.grad)
                p.grad = v if p.dtype == self.grad_dtype else p.grad

    def reduce_gradients(self) -> None:
        """Average the gradients of all replicated trainable parameters across the group (one kernel)."""
        # Experts under expert parallelism: the owner already holds the sum over all source ranks of its
        # expert-parallel group; the global mean needs 1/world and a sum over the replicate dimension.
        for p in self.ep_params:
            if p.grad is None:
                continue
            p.grad.mul_(1.0 / self.world)
            rep = getattr(p, "_fmsb_replicate_group", None)
            if rep is not None and dist.get_world_size(rep) > 1:
                dist.all_reduce(p.grad, group=rep)
        if not self.params:
            return
        self._collect_grads()
        if self.world > 1:
            self.comm.allreduce_(self.bucket, self.bucket_numel, self.grad_dtype, scale=self.grad_scale)
            for p, v in zip(self.params, self._grad_views):
                if p.dtype != self.grad_dtype and p.grad is not None:
                    p.grad.copy_(v)


class ShardedOptimizer:
    """ZeRO-1 step for the engine's replicated parameters.

    ``step()`` = reduce-scatter of the flat gradient bucket with the 1/world scale and the cast to fp32 fused (each
    rank pulls its slice from all peers), AdamW on the fp32 master slice, cast of the updated slice into the flat
    parameter buffer, then a pull all-gather of the other ranks' slices.  Optimizer memory per rank is 12 bytes per
    parameter divided by the world size instead of replicated.  Expert-parallel parameters keep their own optimizer.
    """

    def __init__(self, engine: "ShardedEngine", lr, weight_decay, betas, eps):
        self.engine = engine
        e = engine
        self.master = e.flat_params[e.own_slice].float().clone().requires_grad_(False)
        self.master.grad = torch.zeros_like(self.master)
        self.inner = torch.optim.AdamW([self.master], lr=lr, weight_decay=weight_decay, betas=betas, eps=eps, fused=True)
        self.param_groups = self.inner.param_groups
        self.max_grad_norm = 0.0
        esize = torch.empty((), dtype=e.param_dtype).element_size()
        # rank r's updated slice lives at byte offset r * slice inside ITS OWN flat buffer
        self._slice_bytes = e.n_own * esize
        import ctypes

        self._slice_ptrs = (ctypes.c_void_p * e.world)(*[p + r * self._slice_bytes
                                                         for r, p in enumerate(e.param_bucket.ptrs)])

    def step(self) -> None:
        e = self.engine
        e._collect_grads()
        e.comm.reduce_scatter(e.bucket, e.n_own, e.grad_dtype, self.master.grad, scale=e.grad_scale)
        if self.max_grad_norm and self.max_grad_norm > 0:
            # global norm of the averaged gradient = sqrt of the sum over ranks of the slices' squared norms
            sq = self.master.grad.pow(2).sum()
            dist.all_reduce(sq, group=e.group)
            self.master.grad.mul_(torch.clamp(self.max_grad_norm / (sq.sqrt() + 1e-6), max=1.0))
        self.inner.step()
        e.flat_params[e.own_slice].copy_(self.master)
        e.comm.barrier(6)  # every rank's slice is written
        from .. import _native as NV

        rc = NV.lib().fmsb_comm_allgather(self._slice_ptrs, e.flat_params.data_ptr(), self._slice_bytes, e.rank,
                                          e.world, 32, NV.stream_ptr())
        NV.check(rc, "fmsb_comm_allgather")
        e.comm.barrier(7)  # nobody rewrites a slice that a peer is still pulling

    def zero_grad(self, set_to_none: bool = True) -> None:
        self.engine.zero_grad()

    def state_dict(self):
        return {"inner": self.inner.state_dict(), "master": self.master}

    def load_state_dict(self, sd) -> None:
        self.inner.load_state_dict(sd["inner"])
        self.master.copy_(sd["master"])


def install_engine(model: nn.Module, accelerator, **kwargs) -> Optional[ShardedEngine]:
    """Create the engine once per accelerator when running with more than one process."""
    if getattr(accelerator, "engine", None) is not None:
        return accelerator.engine
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return None
    if os.environ.get("FMSB_SHARD_FROZEN", "1") == "0":
        kwargs["shard_frozen"] = False  # keep the frozen weights replicated (memory for less traffic)
    accelerator.engine = ShardedEngine(model, **kwargs)
    return accelerator.engine
