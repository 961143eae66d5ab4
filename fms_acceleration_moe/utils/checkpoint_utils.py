"""``python -m fms_acceleration_moe.utils.checkpoint_utils <ckpt_dir> <out_dir> [pretrained]``: forwards to
:mod:`fms_acceleration_b200.plugins.moe.utils.checkpoint_utils`."""
import sys

from fms_acceleration_b200.plugins.moe.utils.checkpoint_utils import *  # noqa: F401,F403
from fms_acceleration_b200.plugins.moe.utils.checkpoint_utils import main

if __name__ == "__main__":
    sys.exit(main())
