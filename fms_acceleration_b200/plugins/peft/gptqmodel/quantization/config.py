"""``QuantizeConfig``: the description of a GPTQ quantisation stored beside a checkpoint.

Field names, file names and synonyms follow fms_acceleration_peft/gptqmodel/quantization/config.py:35-321 of
the reference so that existing ``quantize_config.json`` files (and ``config.json["quantization_config"]``
sections) load unchanged.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, fields
from typing import Any, Dict, Optional

QUANT_CONFIG_FILENAME = "quantize_config.json"
QUANT_CONFIG_FILENAME_COMPAT = [QUANT_CONFIG_FILENAME, "quant_config.json", "config.json"]
FORMAT_FIELD_JSON = "checkpoint_format"
FORMAT_FIELD_COMPAT = "format"
QUANT_METHOD_FIELD = "quant_method"
META_FIELD = "meta"
META_FIELD_QUANTIZER = "quantizer"
META_QUANTIZER_NAME = "fms_acceleration_b200"
MIN_VERSION_WITH_V2 = "0.9.0"


class FORMAT:
    GPTQ = "gptq"        # v1: zero points stored minus one
    GPTQ_V2 = "gptq_v2"  # zero points stored as is
    TRITON = "triton"    # alias kept for old checkpoints (v1 layout)


class QUANT_METHOD:
    GPTQ = "gptq"


QUANT_METHOD_FORMAT_MAPPING = {QUANT_METHOD.GPTQ: {FORMAT.GPTQ, FORMAT.GPTQ_V2, FORMAT.TRITON}}

# other libraries' names for the same fields
QUANT_CONFIG_ARG_SYNONYMS = {"w_bit": "bits", "q_group_size": "group_size", FORMAT_FIELD_COMPAT: FORMAT_FIELD_JSON}


@dataclass
class QuantizeConfig:
    bits: int = 4
    group_size: int = -1
    damp_percent: float = 0.01
    desc_act: bool = True
    static_groups: bool = False
    sym: bool = True
    true_sequential: bool = True
    lm_head: bool = False
    quant_method: str = QUANT_METHOD.GPTQ
    format: str = FORMAT.GPTQ
    model_name_or_path: Optional[str] = None
    model_file_base_name: Optional[str] = None
    meta: Optional[Dict[str, Any]] = None

    def __post_init__(self):
        if self.bits not in (2, 3, 4, 8):
            raise ValueError(f"only support quantize to {[2, 3, 4, 8]} bits.")
        if self.group_size != -1 and self.group_size <= 0:
            raise ValueError("unless equal to -1, group_size must greater then 0.")
        if not 0 < self.damp_percent < 1:
            raise ValueError("damp_percent must between 0 and 1.")
        if self.quant_method not in QUANT_METHOD_FORMAT_MAPPING:
            raise ValueError(f"Unsupported quantization method: {self.quant_method}")
        if self.format not in QUANT_METHOD_FORMAT_MAPPING[self.quant_method]:
            raise ValueError(f"format {self.format!r} is not valid for method {self.quant_method!r}")
        if self.meta is None:
            self.meta = {}
        elif not isinstance(self.meta, dict):
            raise ValueError("meta must be a dictionary")

    # -- meta ------------------------------------------------------------------------------------
    def meta_set(self, key: str, value: Any) -> None:
        self.meta[key] = value

    def meta_get(self, key: str) -> Any:
        return self.meta.get(key)

    def meta_set_versionable(self, key: str, value: str, version: str) -> None:
        self.meta_set(key, f"{value}:{version}")

    def meta_get_versionable(self, key: str):
        v = self.meta_get(key)
        if v is None:
            return None, None
        name, _, ver = str(v).partition(":")
        return name.lower(), (ver.lower() or None)

    def is_quantized_or_packed_by_v2(self) -> bool:
        """True when the producer recorded in ``meta`` is known to write the v2 zero-point layout."""
        name, _ = self.meta_get_versionable(META_FIELD_QUANTIZER)
        return name in (META_QUANTIZER_NAME, "gptqmodel")

    # -- (de)serialisation -------------------------------------------------------------------------
    def to_dict(self) -> Dict[str, Any]:
        return {
            "bits": self.bits, "group_size": self.group_size, "desc_act": self.desc_act,
            "static_groups": self.static_groups, "sym": self.sym, "lm_head": self.lm_head,
            "damp_percent": self.damp_percent, "true_sequential": self.true_sequential,
            "model_name_or_path": self.model_name_or_path, "model_file_base_name": self.model_file_base_name,
            QUANT_METHOD_FIELD: self.quant_method, FORMAT_FIELD_JSON: self.format, META_FIELD: self.meta,
        }

    def save_pretrained(self, save_dir: str, **kwargs) -> None:
        with open(os.path.join(save_dir, QUANT_CONFIG_FILENAME), "w", encoding="utf-8") as fh:
            json.dump(self.to_dict(), fh, indent=2)

    @classmethod
    def from_quant_config(cls, quantize_cfg: Dict[str, Any], format: Optional[str] = None) -> "QuantizeConfig":
        valid = {f.name for f in fields(cls)}
        format_auto_inferred = False
        if format is None:
            format_auto_inferred = True
        normalized: Dict[str, Any] = {QUANT_METHOD_FIELD: QUANT_METHOD.GPTQ,
                                      FORMAT_FIELD_JSON: format if format else FORMAT.GPTQ}
        for key, val in quantize_cfg.items():
            key = key.lower()
            key = QUANT_CONFIG_ARG_SYNONYMS.get(key, key)
            if key == FORMAT_FIELD_JSON:
                val = str(val).lower()
                if val in (FORMAT.GPTQ, FORMAT.GPTQ_V2, FORMAT.TRITON):
                    if format is None or format_auto_inferred:
                        normalized[key] = val
                    format_auto_inferred = False
            elif key == QUANT_METHOD_FIELD:
                normalized[key] = str(val).lower()
            elif key in valid:
                normalized[key] = val
        normalized["format"] = normalized.pop(FORMAT_FIELD_JSON)
        return cls(**{k: v for k, v in normalized.items() if k in valid})

    @classmethod
    def from_pretrained(cls, save_dir: str, **kwargs) -> "QuantizeConfig":
        format = kwargs.pop("format", None)
        for name in QUANT_CONFIG_FILENAME_COMPAT:
            path = os.path.join(save_dir, name)
            if not os.path.exists(path):
                continue
            with open(path, encoding="utf-8") as fh:
                raw = json.load(fh)
            if name == "config.json":
                raw = raw.get("quantization_config")
                if raw is None:
                    continue
            return cls.from_quant_config(raw, format)
        raise ValueError(f"No {QUANT_CONFIG_FILENAME_COMPAT} found in {save_dir!r}")


class BaseQuantizeConfig(QuantizeConfig):
    """Earlier name of :class:`QuantizeConfig`, kept as the reference keeps it (quantization/config.py:324-331)."""

    def __init__(self, *args, **kwargs):
        import warnings

        warnings.warn("BaseQuantizeConfig is the earlier name of QuantizeConfig", DeprecationWarning, stacklevel=2)
        super().__init__(*args, **kwargs)
