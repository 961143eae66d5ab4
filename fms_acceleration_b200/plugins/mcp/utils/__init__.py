from .utils import patch_mamba_layers_with_cp_head, hf_config_ssm_config  # noqa: F401
