"""AdamW whose step is one in-tree kernel launch per parameter tensor (``csrc/elementwise.cu: adamw_kernel``).

Drop-in for ``torch.optim.AdamW`` (same constructor, same ``state_dict`` layout: ``step`` / ``exp_avg`` /
``exp_avg_sq`` per parameter, moments in the parameter's dtype), so checkpoints written with either load into the
other.  The arithmetic is that of torch's fused implementation: fp32 math per element, one rounding per stored value.
The reference trains with ``torch.optim.AdamW`` through the Hugging Face trainer (``adamw_torch`` in
scripts/benchmarks/defaults.yaml); torch's multi-tensor kernel reached about half of the copy bandwidth on the
3.3 B parameters of a Granite-3B full fine-tune (14 ms per step).

Parameters that are not dense CUDA tensors of fp16 / bf16 / fp32, or whose gradient has another dtype or layout, take
torch's own single-tensor path.
"""
from __future__ import annotations

import ctypes

import torch

from .. import _native as N

_P, _L, _F, _I = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_float, ctypes.c_int
N.declare("fmsb_adamw", [_P, _P, _P, _P, _L, _F, _F, _F, _F, _F, _F, _F, _F, _I, _P])


class AdamW(torch.optim.AdamW):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=1e-2, **kwargs):
        for k in ("fused", "foreach", "capturable"):
            kwargs.pop(k, None)
        if kwargs.get("amsgrad") or kwargs.get("maximize"):
            raise NotImplementedError("amsgrad / maximize are not offered by the in-tree AdamW")
        # the parent keeps the bookkeeping (param groups, state_dict, add_param_group); its own step is the fallback
        super().__init__(params, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, foreach=False, fused=False)
        self.grad_scale = 1.0  # multiplies every gradient inside the kernel (e.g. a clipping coefficient)

    @staticmethod
    def _native_ok(p: torch.Tensor) -> bool:
        g = p.grad
        return (p.is_cuda and p.dtype in (torch.float16, torch.bfloat16, torch.float32) and p.is_contiguous()
                and g is not None and g.dtype == p.dtype and g.is_contiguous() and not g.is_sparse
                and p.data_ptr() % 16 == 0 and g.data_ptr() % 16 == 0)

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            b1, b2 = group["betas"]
            lr, eps, wd = float(group["lr"]), float(group["eps"]), float(group["weight_decay"])
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if len(st) == 0:
                    st["step"] = torch.tensor(0.0, dtype=torch.float32)
                    st["exp_avg"] = torch.zeros_like(p, memory_format=torch.preserve_format)
                    st["exp_avg_sq"] = torch.zeros_like(p, memory_format=torch.preserve_format)
                step_t = st["step"]
                if step_t.is_cuda:  # a state loaded from a checkpoint of torch's fused optimizer
                    step_t = st["step"] = step_t.detach().cpu().to(torch.float32)
                step_t += 1
                t = float(step_t)
                m, v = st["exp_avg"], st["exp_avg_sq"]
                if (self._native_ok(p) and m.dtype == p.dtype and v.dtype == p.dtype and m.is_contiguous()
                        and v.is_contiguous() and m.data_ptr() % 16 == 0 and v.data_ptr() % 16 == 0):
                    rc = N.lib().fmsb_adamw(p.data_ptr(), p.grad.data_ptr(), m.data_ptr(), v.data_ptr(), p.numel(), lr,
                                            float(b1), float(b2), eps, wd, 1.0 - b1 ** t, 1.0 - b2 ** t,
                                            float(self.grad_scale), N.dtype_code(p.dtype), N.stream_ptr())
                    N.check(rc, "fmsb_adamw")
                else:
                    g = p.grad if self.grad_scale == 1.0 else p.grad * self.grad_scale
                    p.mul_(1.0 - lr * wd)
                    m.lerp_(g.to(m.dtype), 1.0 - b1)
                    v.mul_(b2).addcmul_(g.to(v.dtype), g.to(v.dtype), value=1.0 - b2)
                    denom = (v.sqrt() / (1.0 - b2 ** t) ** 0.5).add_(eps)
                    p.addcdiv_(m, denom, value=-lr / (1.0 - b1 ** t))
        return loss
