"""Function names of the reference's ``triton_utils`` (dequantise, then matmul), bound to the CUDA kernels."""
