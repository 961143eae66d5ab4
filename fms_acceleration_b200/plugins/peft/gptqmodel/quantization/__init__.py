from .config import QuantizeConfig, FORMAT, QUANT_METHOD  # noqa: F401
from .gptq import GPTQ  # noqa: F401
from .quantizer import Quantizer  # noqa: F401
from .config import (FORMAT_FIELD_COMPAT as FORMAT_FIELD_CODE, FORMAT_FIELD_JSON, QUANT_CONFIG_FILENAME,  # noqa: F401,E402
                     QUANT_METHOD_FIELD)
from .config import QuantizeConfig as BaseQuantizeConfig  # noqa: F401,E402
from .quantizer import quantize  # noqa: F401,E402
