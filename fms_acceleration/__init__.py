"""Import-compatible alias of ``fms_acceleration_b200.framework``: code written against the ``fms_acceleration`` package of the reference
keeps working (``import fms_acceleration``, ``from fms_acceleration.<module> import ...``).  The implementation lives in
``fms_acceleration_b200.framework``; the submodules listed below are registered under this package's name."""
import importlib
import sys

_TARGET = "fms_acceleration_b200.framework"
_SUBMODULES = ['constants', 'framework', 'framework_plugin', 'model_patcher', 'accelerator_patcher', 'utils', 'utils.test_utils']

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

# importing the framework also registers every in-tree plugin, in activation order
import fms_acceleration_b200.plugins  # noqa: E402,F401
