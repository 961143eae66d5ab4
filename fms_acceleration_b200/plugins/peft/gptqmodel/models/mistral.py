"""``MistralGPTQ``: the layer layout of this family lives with the others in ``families.py``; this module keeps the
reference's import path (gptqmodel/models/mistral.py)."""
from .families import MistralGPTQ  # noqa: F401
