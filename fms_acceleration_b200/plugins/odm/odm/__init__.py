from .dataset import OnlineMixingDataset  # noqa: F401
from .reward import Reward, compute_reward  # noqa: F401
from .auto_categorizer import AutoCategorizeConfig, DatasetAutoCategorizer  # noqa: F401
