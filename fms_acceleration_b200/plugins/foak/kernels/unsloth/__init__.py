"""``fms_acceleration_foak.kernels.unsloth``: the names of the reference's fast RMSNorm / RoPE / cross-entropy modules.
The implementations are the CUDA kernels of ``fms_acceleration_b200.ops`` (``csrc/elementwise.cu``,
``csrc/cross_entropy.cu``); nothing here is Triton."""
