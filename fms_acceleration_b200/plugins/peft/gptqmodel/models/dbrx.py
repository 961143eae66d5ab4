"""``DbrxGPTQ``: the layer layout of this family lives with the others in ``families.py``; this module keeps the
reference's import path (gptqmodel/models/dbrx.py)."""
from .families import DbrxGPTQ  # noqa: F401
