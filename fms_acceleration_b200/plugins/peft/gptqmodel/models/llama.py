"""``LlamaGPTQ``: the layer layout of this family lives with the others in ``families.py``; this module keeps the
reference's import path (gptqmodel/models/llama.py)."""
from .families import LlamaGPTQ  # noqa: F401
