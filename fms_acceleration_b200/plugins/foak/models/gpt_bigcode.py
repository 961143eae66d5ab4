"""Patch rules of the ``gpt_bigcode`` family under the reference's module name (fms_acceleration_foak/models/gpt_bigcode.py)."""
from functools import partial

from .hf import get_mp_rules as _rules

get_mp_rules = partial(_rules, "gpt_bigcode")
get_mp_rules.__doc__ = "get_mp_rules(base_type, config=None) -> list of ModelPatcherRule for gpt_bigcode"
