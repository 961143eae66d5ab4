from .scattermoe_prepare import prepare_scattermoe  # noqa: F401
from .checkpoint_utils import (patch_huggingface_clip_grad_norm_fsdp2,  # noqa: F401,E402
                               patch_huggingface_fsdp2_load_full_state_dict,
                               patch_huggingface_save_and_load_for_dtensors, patch_prepare_sd_options,
                               recover_safetensors_from_dcp)


def patch_torch_optim_foreach_to_not_apply_to_dtensors() -> int:
    """Take ``DTensor`` out of the tensor types for which ``torch.optim`` uses its multi-tensor ("foreach") kernels,
    so that optimizers fall back to one update per parameter for sharded expert tensors (the reference applies this
    when experts are DTensors, fms_acceleration_moe/utils/__init__.py:33-49).  Returns how many entries were removed;
    harmless to call twice."""
    from torch.optim import optimizer as _opt

    kinds = getattr(_opt, "_foreach_supported_types", None)
    if kinds is None:
        return 0
    keep = [t for t in kinds if t.__name__ != "DTensor"]
    removed = len(kinds) - len(keep)
    kinds[:] = keep
    return removed
