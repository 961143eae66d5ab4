"""Import-compatible alias of ``fms_acceleration_b200.plugins.moe``: code written against the ``fms_acceleration_moe`` package of the reference
keeps working (``import fms_acceleration_moe``, ``from fms_acceleration_moe.<module> import ...``).  The implementation lives in
``fms_acceleration_b200.plugins.moe``; the submodules listed below are registered under this package's name."""
import importlib
import sys

_TARGET = "fms_acceleration_b200.plugins.moe"
_SUBMODULES = ['framework_plugin_scattermoe', 'utils.scattermoe', 'utils.scattermoe_prepare', 'utils.scattermoe_state_dict', 'utils.scattermoe_constants']

_pkg = importlib.import_module(_TARGET)
# any other submodule resolves to the module of the same relative name under the target package
from fms_acceleration_b200.compat.alias import install_alias  # noqa: E402

install_alias(__name__, _TARGET)
globals().update({k: v for k, v in vars(_pkg).items() if not k.startswith("__")})
for _sub in _SUBMODULES:
    try:
        sys.modules[f"{__name__}.{_sub}"] = importlib.import_module(f"{_TARGET}.{_sub}")
    except ImportError:  # an optional dependency of that submodule is missing
        pass
