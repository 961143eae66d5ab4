"""ModelPatcher rules of the fused-ops plugin, one set per architecture.

Rule ids follow the reference (``<arch>-rms``, ``<arch>-qkvo``, ``<arch>-mlp``, ``<arch>-rope``,
``<arch>-cross-ent``, ``<arch>-custom-loss``, ``<arch>-fused-lce``;
fms_acceleration_foak/models/llama.py:54-174 and siblings).  ``zoo`` rules target the in-tree model classes,
the others target Hugging Face ``transformers`` classes and are only produced when those import.
"""
from __future__ import annotations

from typing import List

from ....framework.model_patcher import ModelPatcherRule
from . import hf, zoo


def all_rules(base_type: str, config=None) -> List[ModelPatcherRule]:
    rules: List[ModelPatcherRule] = []
    rules += zoo.get_mp_rules(base_type, config)
    for arch in hf.ARCHS:
        rules += hf.get_mp_rules(arch, base_type, config)
    return rules
