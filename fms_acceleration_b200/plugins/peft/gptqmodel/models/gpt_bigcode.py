"""``GPTBigCodeGPTQ``: the layer layout of this family lives with the others in ``families.py``; this module keeps the
reference's import path (gptqmodel/models/gpt_bigcode.py)."""
from .families import GPTBigCodeGPTQ  # noqa: F401
