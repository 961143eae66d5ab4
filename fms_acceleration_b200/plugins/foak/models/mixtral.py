"""Patch rules of the ``mixtral`` family under the reference's module name (fms_acceleration_foak/models/mixtral.py)."""
from functools import partial

from .hf import get_mp_rules as _rules

get_mp_rules = partial(_rules, "mixtral")
get_mp_rules.__doc__ = "get_mp_rules(base_type, config=None) -> list of ModelPatcherRule for mixtral"
