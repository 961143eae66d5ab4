from .auto import GPTQModel, MODEL_MAP  # noqa: F401
from .base import BaseGPTQModel  # noqa: F401
