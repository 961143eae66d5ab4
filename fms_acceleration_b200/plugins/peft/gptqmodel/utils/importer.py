"""Choice of the ``QuantLinear`` class for a quantisation configuration (role of
fms_acceleration_peft/gptqmodel/utils/importer.py:25-71).  There is one implementation here, the sm_100a layer of
``fms_acceleration_b200.nn.gptq``; ``Backend.TRITON`` (the name the reference's configuration uses) and
``Backend.AUTO`` both select it after the settings have been validated against it."""
from __future__ import annotations

from collections import OrderedDict

from fms_acceleration_b200.nn.gptq import QuantLinear

from ..quantization.config import FORMAT
from .backend import Backend

backend_dict = OrderedDict({Backend.B200: QuantLinear, Backend.TRITON: QuantLinear})
format_dict = {FORMAT.GPTQ: [Backend.B200, Backend.TRITON], FORMAT.GPTQ_V2: [Backend.B200, Backend.TRITON],
               FORMAT.TRITON: [Backend.B200, Backend.TRITON]}


def select_quant_linear(bits: int, group_size: int, desc_act: bool, sym: bool, backend: Backend = Backend.AUTO,
                        format: str = FORMAT.GPTQ_V2, pack: bool = False):
    if format not in format_dict:
        raise NotImplementedError(f"unknown checkpoint format {format!r}")
    if backend == Backend.AUTO:
        for b, cls in backend_dict.items():
            if b in format_dict[format] and cls.validate(bits, group_size, desc_act, sym, raise_error=False) \
                    and (hasattr(cls, "pack") or not pack):
                return cls
        raise NotImplementedError(f"no QuantLinear supports bits={bits}, group_size={group_size}, desc_act={desc_act}, sym={sym}")
    if backend not in backend_dict:
        raise NotImplementedError("Invalid Backend")
    cls = backend_dict[backend]
    cls.validate(bits, group_size, desc_act, sym, raise_error=True)
    return cls
