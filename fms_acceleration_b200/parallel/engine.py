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
                 grad_scale: Optional[float] = None, backend: Optional[str] = None):
        """``backend``: "fused" (default on GPUs) moves data with this package's peer-memory kernels; "library" uses
        the process group's collectives (NCCL / gloo) for the gradient reduction and the parameter all-gather of
        the sharded optimizer - the like-for-like baseline of the fused path, and what runs on CPU ranks."""
        self.model = model
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.device = next(model.parameters()).device
        backend = backend or os.environ.get("FMSB_ENGINE_BACKEND") or ("fused" if self.device.type == "cuda" else "library")
        self.fused = backend == "fused" and self.world > 1
        self.comm = Communicator(self.group, self.device) if self.fused else None
        self.comm_stream = torch.cuda.Stream(self.device) if self.device.type == "cuda" else None
        self.reduce_stream = torch.cuda.Stream(self.device, priority=-1) if self.device.type == "cuda" else None
        self._side: dict = {}
        self._micro = 0
        self._ep_reduced = False
        self.sharded_optimizer: Optional["ShardedOptimizer"] = None
        self.shard_optimizer = shard_optimizer
        self.grad_scale = grad_scale  # None: average (1/world); 1.0: plain sum (context parallelism)
        self.layers = self._find_layers(model)
        self.blobs: List[_LayerBlob] = []
        self.arena: Optional[SymmBuffer] = None
        self.staging: List[torch.Tensor] = []
        self._staged: List[Optional[int]] = [None, None]
        self._ready: List[Optional[torch.cuda.Event]] = [None, None]
        self._released: List[Optional[torch.cuda.Event]] = [None, None]
        if shard_frozen and self.fused and self.layers:
            self._shard_frozen_layers()
        self._setup_grad_bucket(grad_dtype)
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
        """Lay the gradients of all replicated trainable parameters out in one flat buffer, cut into segments in
        the order backward produces them (last layers first).  A segment is reduced across the ranks as soon as its
        last gradient has been accumulated (autograd hook), on a stream of its own, while backward goes on: the
        role of FSDP's per-layer reduce-scatter in the reference (scripts/benchmarks/accelerate.yaml:30) and of its
        per-tensor all-reduce hooks for adapters (fms_acceleration_foak/utils.py:39-43,79-80)."""
        # expert-parallel parameters are not replicated over the whole world: they are reduced separately
        self.ep_params = [p for p in self.model.parameters() if p.requires_grad and getattr(p, "_fmsb_expert_parallel", False)]
        self.params = [p for p in self.model.parameters()
                       if p.requires_grad and not getattr(p, "_fmsb_expert_parallel", False)]
        self.bucket = None
        self.segments: List[_Segment] = []
        self.sync_gradients = True  # False while accumulating micro-batches: hooks count but nothing is reduced
        if not self.params:
            return
        dtype = grad_dtype or self.params[0].dtype
        self.grad_dtype = dtype
        esize = torch.empty((), dtype=dtype).element_size()
        unit = self.world * 16 // esize * 8
        seg_bytes = int(float(os.environ.get("FMSB_GRAD_SEGMENT_MB", "128")) * (1 << 20))
        # segments in backward order; a parameter's position in the flat buffer is its position in that order
        order = list(reversed(self.params))
        off = 0
        cur = _Segment(0)
        for p in order:
            cur.params.append(p)
            cur.numel += p.numel()
            if cur.numel * esize >= seg_bytes:
                cur.numel_padded = _align(cur.numel, unit)
                self.segments.append(cur)
                off += cur.numel_padded
                cur = _Segment(off)
        if cur.params:
            cur.numel_padded = _align(cur.numel, unit)
            self.segments.append(cur)
            off += cur.numel_padded
        self.bucket_numel = off
        if self.world > 1 and self.fused:
            self.bucket = SymmBuffer(self.bucket_numel * esize, self.group, self.device)
            flat = self.bucket.view(0, self.bucket_numel, dtype)
        else:
            flat = torch.zeros(self.bucket_numel, dtype=dtype, device=self.device)
        self.flat_grads = flat
        self._grad_view = {}
        self._seg_of = {}
        for seg in self.segments:
            o = seg.offset
            for p in seg.params:
                v = flat[o: o + p.numel()].view_as(p)
                o += p.numel()
                self._grad_view[p] = v
                self._seg_of[p] = seg
                if p.dtype == dtype:
                    p.grad = v
                p.register_post_accumulate_grad_hook(self._on_grad)
            seg.pending = len(seg.params)
        self._grad_views = [self._grad_view[p] for p in self.params]
        if self.world > 1:
            # replicated parameters must start identical
            for p in self.params:
                dist.broadcast(p.data, src=dist.get_global_rank(self.group, 0), group=self.group)

    def _on_grad(self, p: torch.Tensor) -> None:
        """Autograd hook: the gradient of ``p`` is complete for this backward pass."""
        v = self._grad_view[p]
        g = p.grad
        if g is not None and g.data_ptr() != v.data_ptr():
            if p.dtype == self.grad_dtype:
                v.copy_(g)   # autograd replaced the view by (view + new gradient): take the sum back into the bucket
                p.grad = v
            else:
                v.add_(g)    # bucket in another dtype (zeroed by zero_grad): accumulate, keep the tensor for later
                self._side[p] = g
                p.grad = None
        seg = self._seg_of[p]
        seg.pending -= 1
        if seg.pending == 0 and self.sync_gradients and self.world > 1:
            self._launch_segment(seg)

    def _launch_segment(self, seg: "_Segment") -> None:
        """Reduce one segment on the reduction stream, ordered after everything enqueued so far on the compute
        stream.  Every rank launches the segments in the same order (autograd runs the same graph everywhere)."""
        if seg.launched:
            return
        seg.launched = True
        main = torch.cuda.current_stream(self.device) if self.device.type == "cuda" else None
        if not self.fused:
            view = self.flat_grads[seg.offset: seg.offset + seg.numel_padded]
            scale = 1.0 / self.world if self.grad_scale is None else self.grad_scale
            if self.sharded_optimizer is not None:
                n = seg.numel_padded // self.world
                out = self.sharded_optimizer.grad_slice(seg)
                if dist.get_backend(self.group) == "nccl":
                    tmp = torch.empty(n, dtype=view.dtype, device=view.device)
                    dist.reduce_scatter_tensor(tmp, view, group=self.group)
                else:  # gloo has no reduce-scatter
                    dist.all_reduce(view, group=self.group)
                    tmp = view[self.rank * n: (self.rank + 1) * n]
                out.copy_(tmp.float() * scale)
            else:
                dist.all_reduce(view, group=self.group)
                view.mul_(scale)
            return
        ev = torch.cuda.Event()
        ev.record(main)
        with torch.cuda.stream(self.reduce_stream):
            self.reduce_stream.wait_event(ev)
            esize = self.flat_grads.element_size()
            ptrs = self.bucket.ptr_array(seg.offset * esize)
            if self.sharded_optimizer is not None:
                self.comm.reduce_scatter_ptrs(ptrs, seg.numel_padded // self.world, self.grad_dtype,
                                              self.sharded_optimizer.grad_slice(seg), scale=self.grad_scale)
            else:
                mc = self.bucket.mc_ptr + seg.offset * esize if self.bucket.mc_ptr else 0
                self.comm.allreduce_ptrs(ptrs, seg.numel_padded, self.grad_dtype, scale=self.grad_scale, mc_ptr=mc)
            seg.done = torch.cuda.Event()
            seg.done.record(self.reduce_stream)

    # ------------------------------------------------------------------ optimizer state sharding (ZeRO-1)
    def _setup_param_bucket(self) -> None:
        """Replicated trainable parameters become views into one flat symmetric buffer, laid out like the gradient
        bucket, so that rank r can update its slice of every segment and everybody can pull the updated slices."""
        dtypes = {p.dtype for p in self.params}
        if len(dtypes) != 1:
            raise ValueError("optimizer sharding needs all replicated trainable parameters in one dtype")
        self.param_dtype = dtypes.pop()
        esize = torch.empty((), dtype=self.param_dtype).element_size()
        if self.fused:
            self.param_bucket = SymmBuffer(self.bucket_numel * esize, self.group, self.device)
            flat = self.param_bucket.view(0, self.bucket_numel, self.param_dtype)
        else:
            self.param_bucket = None
            flat = torch.zeros(self.bucket_numel, dtype=self.param_dtype, device=self.device)
        with torch.no_grad():
            for seg in self.segments:
                o = seg.offset
                for p in seg.params:
                    v = flat[o: o + p.numel()].view_as(p)
                    v.copy_(p.data)
                    p.data = v
                    o += p.numel()
        self.flat_params = flat
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        dist.barrier(self.group)

    def build_optimizer(self, lr: float, weight_decay: float = 0.0, betas=(0.9, 0.999), eps: float = 1e-8):
        """AdamW over this rank's 1/world slice of every segment (fp32 master copy and moments)."""
        if not hasattr(self, "flat_params"):
            raise RuntimeError("the engine was created without shard_optimizer=True (or runs on one rank)")
        self.sharded_optimizer = ShardedOptimizer(self, lr, weight_decay, betas, eps)
        return self.sharded_optimizer

    def zero_grad(self) -> None:
        self._ep_reduced = False
        for p in self.ep_params:
            p.grad = None
        if not self.params:
            return
        self.flat_grads.zero_()
        for p in self.params:
            p.grad = self._grad_view[p] if p.dtype == self.grad_dtype else None
        for seg in self.segments:
            seg.pending = len(seg.params)
            seg.launched = False
            seg.done = None
        self._micro = 0

    def begin_micro_step(self, last: bool) -> None:
        """Call before the backward pass of every micro-batch: only the last one of an accumulation window reduces."""
        self.sync_gradients = bool(last)
        for seg in self.segments:
            seg.pending = len(seg.params)

    def end_micro_step(self) -> None:
        self._micro += 1

    def reduce_gradients(self) -> None:
        """Finish the gradient reduction of this step: launch the segments that backward did not complete (parameters
        without a gradient this step), make the compute stream wait for all of them, and reduce the expert-parallel
        parameters over their replicate group."""
        # Experts under expert parallelism: the owner already holds the sum over all source ranks of its
        # expert-parallel group; the global mean needs 1/world and a sum over the replicate dimension.
        if not self._ep_reduced:
            self._ep_reduced = True
            for p in self.ep_params:
                if p.grad is None:
                    continue
                p.grad.mul_(1.0 / self.world)
                rep = getattr(p, "_fmsb_replicate_group", None)
                if rep is not None and dist.get_world_size(rep) > 1:
                    dist.all_reduce(p.grad, group=rep)
        if not self.params:
            return
        if self.world > 1:
            for seg in self.segments:
                self._launch_segment(seg)
            if self.fused:
                main = torch.cuda.current_stream(self.device)
                for seg in self.segments:
                    if seg.done is not None:
                        main.wait_event(seg.done)
        if self.sharded_optimizer is None:
            for p, g in self._side.items():  # parameters whose dtype differs from the bucket's
                g.copy_(self._grad_view[p])
                p.grad = g
            self._side = {}


class _Segment:
    """A run of parameters whose gradients are reduced together."""

    def __init__(self, offset: int):
        self.offset = offset       # first element in the flat buffers
        self.numel = 0
        self.numel_padded = 0      # multiple of world * 16 bytes * 8
        self.params: List[torch.Tensor] = []
        self.pending = 0
        self.launched = False
        self.done = None
        self.master_offset = 0     # first element of this rank's slice inside the sharded optimizer's master copy


class ShardedOptimizer:
    """ZeRO-1 step for the engine's replicated parameters.

    During backward every segment of the flat gradient bucket is reduce-scattered (each rank pulls its 1/world of
    the segment from all peers, 1/world scale and the cast to fp32 fused) as soon as the segment's gradients are
    complete.  ``step()`` = AdamW on the fp32 master slices, cast of the updated slices into the flat parameter
    buffer, then a pull all-gather of the other ranks' slices.  Optimizer memory per rank is 12 bytes per parameter
    divided by the world size instead of replicated.  Expert-parallel parameters keep their own optimizer
    (``ep_optimizer``), stepped together with this one.
    """

    def __init__(self, engine: "ShardedEngine", lr, weight_decay, betas, eps):
        self.engine = engine
        e = engine
        moff = 0
        for seg in e.segments:
            seg.master_offset = moff
            moff += seg.numel_padded // e.world
        self.n_master = moff
        self.master = torch.empty(moff, dtype=torch.float32, device=e.device)
        for seg in e.segments:
            self._master_slice(seg).copy_(self._param_slice(seg))
        self.master.grad = torch.zeros_like(self.master)
        self.inner = torch.optim.AdamW([self.master], lr=lr, weight_decay=weight_decay, betas=betas, eps=eps,
                                       fused=e.device.type == "cuda")
        self.param_groups = self.inner.param_groups
        self.max_grad_norm = 0.0
        self.ep_optimizer: Optional[torch.optim.Optimizer] = None
        self.last_grad_norm: Optional[torch.Tensor] = None

    def _own(self, seg: "_Segment"):
        n = seg.numel_padded // self.engine.world
        return seg.offset + self.engine.rank * n, n

    def _param_slice(self, seg) -> torch.Tensor:
        o, n = self._own(seg)
        return self.engine.flat_params[o: o + n]

    def _master_slice(self, seg) -> torch.Tensor:
        return self.master[seg.master_offset: seg.master_offset + seg.numel_padded // self.engine.world]

    def grad_slice(self, seg) -> torch.Tensor:
        """Where the reduce-scatter of ``seg`` puts this rank's part of the averaged gradient (fp32)."""
        return self.master.grad[seg.master_offset: seg.master_offset + seg.numel_padded // self.engine.world]

    def step(self) -> None:
        e = self.engine
        e.reduce_gradients()  # no-op for segments already reduced during backward; waits for all of them
        if self.max_grad_norm and self.max_grad_norm > 0:
            # global norm of the averaged gradient = sqrt of the sum over ranks of the slices' squared norms, plus the
            # expert shards (disjoint over the expert-parallel ranks, replicated over the replicate dimension)
            sq = self.master.grad.pow(2).sum()
            if e.ep_params:
                esq = torch.stack([p.grad.float().pow(2).sum() for p in e.ep_params if p.grad is not None]).sum()
                rep = getattr(e.ep_params[0], "_fmsb_replicate_group", None)
                n_rep = dist.get_world_size(rep) if rep is not None else 1
                sq = sq + esq / n_rep
            dist.all_reduce(sq, group=e.group)
            norm = sq.sqrt()
            coef = torch.clamp(self.max_grad_norm / (norm + 1e-6), max=1.0)
            self.master.grad.mul_(coef)
            for p in e.ep_params:
                if p.grad is not None:
                    p.grad.mul_(coef.to(p.grad.dtype))
            self.last_grad_norm = norm
        self.inner.step()
        if self.ep_optimizer is not None:
            self.ep_optimizer.step()
        for seg in e.segments:
            self._param_slice(seg).copy_(self._master_slice(seg))
        if e.world == 1:
            return
        if not e.fused:
            self._allgather_library()
            return
        e.comm.barrier(6)  # every rank's slices are written
        from .. import _native as NV

        esize = e.flat_params.element_size()
        for seg in e.segments:
            n = seg.numel_padded // e.world
            ptrs = e.param_bucket.ptr_array_strided(seg.offset * esize, n * esize)
            # after the optimizer step nothing else runs: give the pull most of the SMs
            rc = NV.lib().fmsb_comm_allgather(ptrs, e.flat_params.data_ptr() + seg.offset * esize, n * esize, e.rank,
                                              e.world, 96, NV.stream_ptr())
            NV.check(rc, "fmsb_comm_allgather")
        e.comm.barrier(7)  # nobody rewrites a slice that a peer is still pulling

    def zero_grad(self, set_to_none: bool = True) -> None:
        self.engine.zero_grad()
        if self.ep_optimizer is not None:
            self.ep_optimizer.zero_grad(set_to_none=True)

    # plain (per-rank) form
    def state_dict(self):
        return {"inner": self.inner.state_dict(), "master": self.master}

    def load_state_dict(self, sd) -> None:
        self.inner.load_state_dict(sd["inner"])
        self.master.copy_(sd["master"])
        self._publish_master()

    def _publish_master(self) -> None:
        """After a resume: the flat parameters are rebuilt from the fp32 master slices of all ranks."""
        e = self.engine
        for seg in e.segments:
            self._param_slice(seg).copy_(self._master_slice(seg))
        if e.world > 1:
            if e.fused:
                torch.cuda.synchronize(e.device)
            dist.barrier(e.group)
            self._allgather_library()

    def _allgather_library(self) -> None:
        e = self.engine
        for seg in e.segments:
            n = seg.numel_padded // e.world
            full = e.flat_params[seg.offset: seg.offset + seg.numel_padded]
            dist.all_gather([full[r * n: (r + 1) * n] for r in range(e.world)], self._param_slice(seg).clone(),
                            group=e.group)

    # checkpoint form: every rank's slices as shards of tensors that span the group, so that one
    # torch.distributed.checkpoint directory holds the whole optimizer (cf. the sharded optimizer state the
    # reference gets from FSDP, fms_acceleration_moe/utils/checkpoint_utils.py:107-158)
    def _moments(self):
        st = self.inner.state.get(self.master)
        if not st:
            # a fresh optimizer: create the moments with one step at learning rate 0 on zero gradients
            saved = [g["lr"] for g in self.inner.param_groups]
            for g in self.inner.param_groups:
                g["lr"] = 0.0
            self.master.grad.zero_()
            self.inner.step()
            for g, lr in zip(self.inner.param_groups, saved):
                g["lr"] = lr
            st = self.inner.state[self.master]
            if torch.is_tensor(st.get("step")):
                st["step"].zero_()
        return st

    def sharded_state_dict(self):
        from torch.distributed.device_mesh import DeviceMesh
        from torch.distributed.tensor import DTensor, Shard

        e = self.engine
        st = self._moments()
        out = {"step": st["step"].detach().clone().cpu() if torch.is_tensor(st["step"]) else torch.tensor(float(st["step"]))}
        if e.world == 1:
            out.update({"master": self.master, "exp_avg": st["exp_avg"], "exp_avg_sq": st["exp_avg_sq"]})
        else:
            if not hasattr(self, "_mesh"):
                self._mesh = DeviceMesh.from_group(e.group, e.device.type)
            for i, seg in enumerate(e.segments):
                lo, n = seg.master_offset, seg.numel_padded // e.world
                for name, t in (("master", self.master), ("exp_avg", st["exp_avg"]), ("exp_avg_sq", st["exp_avg_sq"])):
                    out[f"{name}.{i}"] = DTensor.from_local(t[lo: lo + n], self._mesh, [Shard(0)], run_check=False)
        if self.ep_optimizer is not None:
            from ..plugins.moe.utils.checkpoint_utils import _optimizer_state

            out["experts"] = _optimizer_state(self.ep_optimizer, e.model)
        return out

    def load_sharded_state_dict(self, sd) -> None:
        """``sd`` is what :meth:`sharded_state_dict` returned after the checkpoint reader filled it in place."""
        st = self._moments()
        if torch.is_tensor(st["step"]):
            st["step"].copy_(sd["step"].to(st["step"].device))
        else:
            st["step"] = float(sd["step"])
        if self.ep_optimizer is not None and "experts" in sd:
            from ..plugins.moe.utils.checkpoint_utils import _unwrap_optimizer_state

            self.ep_optimizer.load_state_dict(_unwrap_optimizer_state(sd["experts"]))
        self._publish_master()


def install_engine(model: nn.Module, accelerator, **kwargs) -> Optional[ShardedEngine]:
    """Create the engine once per accelerator when running with more than one process."""
    if getattr(accelerator, "engine", None) is not None:
        return accelerator.engine
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return None
    if os.environ.get("FMSB_SHARD_FROZEN", "1") == "0":
        kwargs["shard_frozen"] = False  # keep the frozen weights replicated (memory for less traffic)
    if "shard_optimizer" not in kwargs:
        # a full fine-tune: every rank would hold 12 bytes of AdamW state per replicated parameter; shard them over the
        # ranks (reduce-scatter during backward, step on 1/world, all-gather), as FSDP does for the reference.  Adapter
        # runs keep the replicated optimizer: their state is a few hundred MB and the all-gather would not pay.
        full_ft = not any("lora_" in n for n, p in model.named_parameters() if p.requires_grad)
        kwargs["shard_optimizer"] = full_ft and os.environ.get("FMSB_ZERO1", "1") != "0"
    accelerator.engine = ShardedEngine(model, **kwargs)
    return accelerator.engine
