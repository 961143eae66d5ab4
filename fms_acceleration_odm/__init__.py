"""Import-compatible alias of ``fms_acceleration_b200.plugins.odm``: code written against the ``fms_acceleration_odm`` package of the reference
keeps working (``import fms_acceleration_odm``, ``from fms_acceleration_odm.<module> import ...``).  The implementation lives in
``fms_acceleration_b200.plugins.odm``; the submodules listed below are registered under this package's name."""
import importlib
import sys

_TARGET = "fms_acceleration_b200.plugins.odm"
_SUBMODULES = ['framework_plugin_odm', 'odm', 'odm.dataset', 'odm.reward', 'odm.auto_categorizer', 'callback', 'patch']

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
