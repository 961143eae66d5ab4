"""The name the reference's loader imports its layer from
(fms_acceleration_peft/gptqmodel/nn_modules/qlinear/qlinear_tritonv2.py:34-226).  Here it is the sm_100a layer:
dequantise kernel + tcgen05 GEMM, no Triton."""
from fms_acceleration_b200.nn.gptq import QuantLinear  # noqa: F401

__all__ = ["QuantLinear"]
