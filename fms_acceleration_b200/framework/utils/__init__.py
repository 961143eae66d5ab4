"""Helpers shipped with the framework: the testing utilities are importable from the package itself
(``from fms_acceleration.utils import instantiate_framework, read_configuration``), as in the reference
(fms_acceleration/utils/__init__.py:16)."""
from .test_utils import *  # noqa: F401,F403
