"""``GPTQuantLinear``: an ``nn.Linear``-shaped view of a packed GPTQ layer, so that code which looks for linear
layers (adapter installation, module walkers) finds it (the reference's
fms_acceleration_foak/fused_ops/unsloth_lora/gptq/triton/layers.py:28-172).  It shares the packed tensors of the
layer it is built from and multiplies through the dequantisation kernel and the tensor-core GEMM."""
from __future__ import annotations

import torch
from torch import nn

from fms_acceleration_b200.plugins.peft.gptqmodel.nn_modules.triton_utils.kernels import (
    QuantLinearFunction, QuantLinearInferenceOnlyFunction)


class GPTQuantLinear(nn.Linear):
    QUANT_TYPE = "cuda"

    def __init__(self, quant_linear_module, trainable: bool = True):
        src = getattr(quant_linear_module, "base_layer", quant_linear_module)
        src_bias = getattr(src, "bias", None)
        has_bias = src_bias is not None and bool(src_bias.count_nonzero() > 0)
        # the dense weight of nn.Linear is never allocated: the parameter aliases the packed tensor
        nn.Module.__init__(self)
        self.in_features = self.infeatures = src.infeatures
        self.out_features = self.outfeatures = src.outfeatures
        self.bits, self.group_size = src.bits, src.group_size
        self.maxq = getattr(src, "maxq", 2 ** src.bits - 1)
        self.weight = nn.Parameter(src.qweight, requires_grad=False)
        self.bias = nn.Parameter(src_bias.data, requires_grad=False) if has_bias else None
        for name in ("qweight", "qzeros", "scales", "g_idx"):
            self.register_buffer(name, getattr(src, name))
        self.trainable = trainable

    def forward(self, x):
        fn = QuantLinearFunction if self.trainable else QuantLinearInferenceOnlyFunction
        out = fn.apply(x.reshape(-1, x.shape[-1]), self.qweight, self.scales, self.qzeros, self.g_idx, self.bits, self.maxq)
        out = out.to(x.dtype).reshape(*x.shape[:-1], self.outfeatures)
        return out + self.bias if self.bias is not None else out

    @classmethod
    def warmup(cls, model, transpose: bool = True, seqlen: int = 2048):
        """Nothing to tune: tile shapes follow from the problem size."""
        return None

    @classmethod
    def inject_to_model(cls, model, target_module_type, **kwargs) -> int:
        """Replace every ``target_module_type`` layer of ``model`` by a :class:`GPTQuantLinear` over the same packed
        tensors; returns how many were replaced."""
        count = 0
        for name, m in list(model.named_modules()):
            if not isinstance(m, target_module_type) or isinstance(m, cls):
                continue
            parent_name, _, child = name.rpartition(".")
            setattr(model.get_submodule(parent_name) if parent_name else model, child, cls(m, **kwargs))
            count += 1
        return count
