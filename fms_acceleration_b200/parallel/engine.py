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
        for p, v in zip(self.params, self._grad_views):
            if p.grad is not None and p.grad.data_ptr() != v.data_ptr():
                v.copy_(p.grad)
                p.grad = v if p.dtype == self.grad_dtype else p.grad
        if self.world > 1:
            self.comm.allreduce_(self.bucket, self.bucket_numel, self.grad_dtype, scale=self.grad_scale)
            for p, v in zip(self.params, self._grad_views):
                if p.dtype != self.grad_dtype and p.grad is not None:
                    p.grad.copy_(v)


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
