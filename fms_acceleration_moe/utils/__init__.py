"""Alias of :mod:`fms_acceleration_b200.plugins.moe.utils`."""
from fms_acceleration_b200.plugins.moe.utils import *  # noqa: F401,F403
from fms_acceleration_b200.plugins.moe.utils import prepare_scattermoe  # noqa: F401
