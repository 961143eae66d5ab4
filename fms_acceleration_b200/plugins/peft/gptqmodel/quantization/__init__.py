from .config import QuantizeConfig, FORMAT, QUANT_METHOD  # noqa: F401
from .gptq import GPTQ  # noqa: F401
from .quantizer import Quantizer  # noqa: F401
