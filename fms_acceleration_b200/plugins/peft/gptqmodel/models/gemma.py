"""``GemmaGPTQ``: the layer layout of this family lives with the others in ``families.py``; this module keeps the
reference's import path (gptqmodel/models/gemma.py)."""
from .families import GemmaGPTQ  # noqa: F401
