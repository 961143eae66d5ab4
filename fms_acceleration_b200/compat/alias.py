"""Alias packages: ``import fms_acceleration_foak.kernels.unsloth.rms_layernorm`` has to give the module that lives
at ``fms_acceleration_b200.plugins.foak.kernels.unsloth.rms_layernorm`` (the same object, not a second copy whose
relative imports would point outside its package).  :func:`install_alias` puts a finder on ``sys.meta_path`` that
resolves every submodule of the alias to the module of the same relative name under the target package."""
from __future__ import annotations

import importlib
import importlib.abc
import importlib.machinery
import importlib.util
import sys


class _AliasFinder(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    def __init__(self, alias: str, target: str):
        self.alias, self.target = alias, target

    def _real(self, fullname: str) -> str:
        return self.target + fullname[len(self.alias):]

    def find_spec(self, fullname, path=None, target=None):
        if not fullname.startswith(self.alias + "."):
            return None
        try:
            real_spec = importlib.util.find_spec(self._real(fullname))
        except (ImportError, ValueError):
            return None
        if real_spec is None:
            return None
        return importlib.machinery.ModuleSpec(fullname, self, is_package=real_spec.submodule_search_locations is not None)

    def create_module(self, spec):
        return importlib.import_module(self._real(spec.name))  # the one and only module object

    def exec_module(self, module):  # already executed under its real name
        return None

    def get_code(self, fullname):
        """For ``python -m <alias>.<module>``: run the real module as ``__main__`` under its real name, so that its
        relative imports resolve inside the package it lives in."""
        real = self._real(fullname)
        src = f"import runpy\nrunpy.run_module({real!r}, run_name='__main__', alter_sys=True)\n"
        return compile(src, f"<alias of {real}>", "exec")


def install_alias(alias: str, target: str) -> None:
    for f in sys.meta_path:
        if isinstance(f, _AliasFinder) and f.alias == alias:
            return
    sys.meta_path.insert(0, _AliasFinder(alias, target))
