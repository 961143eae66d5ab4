"""Constants shared by the per-family GPTQ model descriptions (the reference's gptqmodel/models/_const.py:18-35)."""
from torch import device

from .auto import MODEL_MAP

CPU = device("cpu")
CUDA_0 = device("cuda:0")

#: model types a quantised checkpoint can be loaded for
SUPPORTED_MODELS = [m for m in MODEL_MAP if m != "dbrx"]  # stock DBRX has to be converted first

#: default longest input of the ExLlama back-ends of other GPTQ libraries; carried for configuration compatibility
EXLLAMA_DEFAULT_MAX_INPUT_LENGTH = 2048

#: placeholder in a layer-module path that stands for the index of one expert
EXPERT_INDEX_PLACEHOLDER = "{expert_index}"
