from .auto import GPTQModel, MODEL_MAP  # noqa: F401
from .base import BaseGPTQModel  # noqa: F401
from .families import (DbrxConvertedGPTQ, DbrxGPTQ, GemmaGPTQ, GPTBigCodeGPTQ, GPTNeoXGPTQ, GraniteGPTQ,  # noqa: F401,E402
                       LlamaGPTQ, MistralGPTQ, MixtralGPTQ)
