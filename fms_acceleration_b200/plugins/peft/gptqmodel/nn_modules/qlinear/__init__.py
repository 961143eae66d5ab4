"""``BaseQuantLinear`` of the reference (fms_acceleration_peft/gptqmodel/nn_modules/qlinear/__init__.py:1-51) is the
in-tree ``QuantLinear``: it carries the ``SUPPORTED_*`` tables and ``validate`` itself."""
from fms_acceleration_b200.nn.gptq import QuantLinear as BaseQuantLinear  # noqa: F401

BaseCudaQuantLinear = BaseQuantLinear
