"""Library-collective baseline of expert parallelism (role of the reference's
fms_acceleration_moe/utils/scattermoe_utils/expert_parallel.py:97-232).

The training path of this repository moves expert rows with its own kernels over peer memory (``ops/moe.py``,
``csrc/moe.cu``).  These two functions do the same exchange with ``torch.distributed.all_to_all_single`` (NCCL on
GPUs, gloo on CPUs): the baseline the fused kernels are compared with, and a CPU-testable statement of what they
have to compute."""
from .expert_parallel import all_to_all_gather_inputs, scatter_with_routing_weights  # noqa: F401
