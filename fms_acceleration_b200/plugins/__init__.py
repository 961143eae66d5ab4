"""The six acceleration plugins.  Importing this package imports them in activation order (loaders first),
which registers them with the framework - the in-tree equivalent of the reference's import-time discovery of
installed ``fms_acceleration_<name>`` packages (fms_acceleration/__init__.py:28-31)."""
import importlib

from ..framework.constants import PLUGINS

for _name in PLUGINS:
    importlib.import_module(f"{__name__}.{_name}")
