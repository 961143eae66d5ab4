"""``python -m fms_acceleration.cli``: forwards to :mod:`fms_acceleration_b200.framework.cli`."""
import sys

from fms_acceleration_b200.framework.cli import *  # noqa: F401,F403
from fms_acceleration_b200.framework.cli import cli

if __name__ == "__main__":
    sys.exit(cli())
