"""Kernel back-ends a GPTQ model can be loaded with.  ``TRITON`` is accepted for configuration compatibility
with the reference (fms_acceleration_peft/gptqmodel/utils/backend.py:20-29) and maps to the CUDA path."""
from enum import Enum


class Backend(Enum):
    AUTO = 0
    TRITON = 1
    B200 = 2


def get_backend(name: str) -> Backend:
    try:
        return Backend[name.upper()]
    except KeyError as exc:
        raise ValueError(f"unknown backend {name!r}") from exc
