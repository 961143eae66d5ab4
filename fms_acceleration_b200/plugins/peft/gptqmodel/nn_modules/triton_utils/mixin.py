"""``TritonModuleMixin``: the warm-up hook of kernel classes that tune themselves on first use
(fms_acceleration_peft/gptqmodel/nn_modules/triton_utils/mixin.py:16-19).  The CUDA kernels of this package pick
their tile shape from the problem size at launch and have nothing to tune, so the hook does nothing."""


class TritonModuleMixin:
    @classmethod
    def warmup(cls, model, transpose: bool = False, seqlen: int = 2048):
        return None
