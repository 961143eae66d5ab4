"""``fms_acceleration_foak.fused_ops.unsloth_lora``: fused LoRA projections and gated activations.  The reference's
three autograd functions per base type (``LoRA_QKV``, ``LoRA_W``, ``LoRA_MLP``) are one mechanism here, the
projection group of ``fms_acceleration_b200.ops.proj``."""
from .geglu import (geglu_approx_backward_kernel, geglu_approx_forward_kernel, geglu_exact_backward_kernel,  # noqa: F401,E402
                    geglu_exact_forward_kernel)
from .swiglu import swiglu_DWf_DW_dfg_kernel, swiglu_fg_kernel  # noqa: F401,E402
from .utils import QUANT_STATE, fast_dequantize, fast_gemv, fast_linear_forward, matmul_lora  # noqa: F401,E402
