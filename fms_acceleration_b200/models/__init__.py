"""Model zoo with HF-compatible module and parameter names (no hub access needed)."""
from .config import DecoderConfig, PRESETS, preset  # noqa: F401
from .llama import LlamaForCausalLM, CausalLMOutput  # noqa: F401
