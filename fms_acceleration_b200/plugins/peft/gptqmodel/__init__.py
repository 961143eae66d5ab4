"""In-tree GPTQ library: quantise, pack, save and load 2/4/8-bit GPTQ models (role of the reference's
fms_acceleration_peft/gptqmodel package)."""
from .models.auto import GPTQModel  # noqa: F401
from .models.base import BaseGPTQModel  # noqa: F401
from .quantization.config import QuantizeConfig, FORMAT, QUANT_METHOD  # noqa: F401
from .utils.backend import Backend  # noqa: F401
