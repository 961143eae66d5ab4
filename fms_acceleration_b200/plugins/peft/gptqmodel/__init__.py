"""In-tree GPTQ library: quantise, pack, save and load 2/4/8-bit GPTQ models (role of the reference's
fms_acceleration_peft/gptqmodel package)."""
from .models.auto import GPTQModel  # noqa: F401
from .models.base import BaseGPTQModel  # noqa: F401
from .quantization.config import QuantizeConfig, FORMAT, QUANT_METHOD  # noqa: F401
from .utils.backend import Backend  # noqa: F401
from .quantization.config import QuantizeConfig as BaseQuantizeConfig  # noqa: F401,E402  (older name of the same class)
from .utils.backend import get_backend  # noqa: F401,E402
