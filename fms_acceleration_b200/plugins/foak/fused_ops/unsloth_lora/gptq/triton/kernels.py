"""Names of fms_acceleration_foak/fused_ops/unsloth_lora/gptq/triton/kernels.py:15-153."""
import torch

from fms_acceleration_b200.ops import quant as Q


def dequant_ref(qstate) -> torch.Tensor:
    """PyTorch statement of the dequantisation (oracle)."""
    return Q.gptq_dequant_ref(qstate.qweight, qstate.scales, qstate.qzeros, qstate.g_idx, qstate.bits,
                              getattr(qstate, "zero_offset", 0)).to(qstate.scales.dtype)


def dequant248(qweight, scales, qzeros, g_idx, bits, maxq=None, zero_offset: int = 0) -> torch.Tensor:
    """Dense ``[in, out]`` weight in the dtype of ``scales``."""
    if not qweight.is_cuda:
        return Q.gptq_dequant_ref(qweight, scales, qzeros, g_idx, bits, zero_offset).to(scales.dtype)
    group_size = qweight.shape[0] * 32 // bits // scales.shape[0]
    return Q.gptq_dequant(qweight, scales, qzeros, g_idx, bits, group_size, zero_offset)
