"""``GPTNeoXGPTQ``: the layer layout of this family lives with the others in ``families.py``; this module keeps the
reference's import path (gptqmodel/models/gpt_neox.py)."""
from .families import GPTNeoXGPTQ  # noqa: F401
