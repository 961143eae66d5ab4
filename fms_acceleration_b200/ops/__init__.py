"""Operator front-ends.  CUDA tensors run the hand-written sm_100a kernels of ``csrc/``; CPU tensors
run the plain PyTorch oracles that the numerics tests compare the kernels against."""
