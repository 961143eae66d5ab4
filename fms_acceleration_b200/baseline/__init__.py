"""Same-box comparison arm: the in-tree models executed through library kernels (cuBLAS ``torch.matmul``, the
installed flash-attn, NCCL collectives) and the reference project's own Triton kernels loaded by file path.

This is NOT the reference run through its public API (that needs ``peft``, ``accelerate``, ``trl`` and
``bitsandbytes``, none of which is installable without a network); it is what the reference's hot path reduces to on
this machine, driven by the same models, data and optimizer as the product path, so that the two numbers differ only
in the kernels and the communication engine."""
from .backend import BaselineRunner, reference_kernels_status  # noqa: F401
