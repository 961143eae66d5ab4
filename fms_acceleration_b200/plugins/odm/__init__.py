"""Online data mixing: a multi-armed bandit re-weights dataset categories during training."""
from .framework_plugin_odm import OnlineDataMixingAccelerationPlugin  # noqa: F401
from .odm import OnlineMixingDataset, Reward, compute_reward  # noqa: F401
