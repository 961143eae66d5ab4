"""``DbrxConvertedGPTQ``: the layer layout of this family lives with the others in ``families.py``; this module keeps the
reference's import path (gptqmodel/models/dbrx_converted.py)."""
from .families import DbrxConvertedGPTQ  # noqa: F401
