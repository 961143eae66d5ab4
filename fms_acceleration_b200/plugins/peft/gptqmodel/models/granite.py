"""``GraniteGPTQ``: the layer layout of this family lives with the others in ``families.py``; this module keeps the
reference's import path (gptqmodel/models/granite.py)."""
from .families import GraniteGPTQ  # noqa: F401
