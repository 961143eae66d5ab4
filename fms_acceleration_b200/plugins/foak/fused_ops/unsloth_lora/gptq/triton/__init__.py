"""GPTQ dequantisation under the reference's module name; the kernel is CUDA (``csrc/quant.cu``)."""
