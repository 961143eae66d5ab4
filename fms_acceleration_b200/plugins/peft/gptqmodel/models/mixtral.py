"""``MixtralGPTQ``: the layer layout of this family lives with the others in ``families.py``; this module keeps the
reference's import path (gptqmodel/models/mixtral.py)."""
from .families import MixtralGPTQ  # noqa: F401
