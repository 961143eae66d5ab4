"""Patch rules of the ``granite`` family under the reference's module name (fms_acceleration_foak/models/granite.py)."""
from functools import partial

from .hf import get_mp_rules as _rules

get_mp_rules = partial(_rules, "granite")
get_mp_rules.__doc__ = "get_mp_rules(base_type, config=None) -> list of ModelPatcherRule for granite"
