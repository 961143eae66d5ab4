"""Patch rules of the ``granitemoe`` family under the reference's module name (fms_acceleration_foak/models/granitemoe.py)."""
from functools import partial

from .hf import get_mp_rules as _rules

get_mp_rules = partial(_rules, "granitemoe")
get_mp_rules.__doc__ = "get_mp_rules(base_type, config=None) -> list of ModelPatcherRule for granitemoe"
