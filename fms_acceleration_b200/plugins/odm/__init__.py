"""Online data mixing: a multi-armed bandit re-weights dataset categories during training."""
from .framework_plugin_odm import OnlineDataMixingAccelerationPlugin  # noqa: F401
from .odm import OnlineMixingDataset, Reward, compute_reward  # noqa: F401
from .callback import DataloaderSavingCallback  # noqa: F401,E402
from .patch import patch_hf_trainer_evaluate  # noqa: F401,E402
