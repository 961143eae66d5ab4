"""Plugin base class and registry.

Behavioural contract of fms_acceleration/framework_plugin.py:28-233 in the reference:

* ``AccelerationPlugin.register_plugin(cls, configuration_and_paths=[...], configuration_or_paths=[...])``
  appends to the global ``PLUGIN_REGISTRATIONS`` (registration order is activation order);
* ``get_relevant_configuration_sections(config)`` returns ``[(sub_config, plugin_cls), ...]`` for every
  registration whose AND paths are all present or any of whose OR paths is present; the sub-config is the
  union of the matched sub-trees re-rooted at their full key paths;
* the ``_check_config_*`` validators raise ``AccelerationPluginConfigError`` with messages that name the
  plugin class, the key and the offending value.
"""
from __future__ import annotations

import importlib.metadata
import sys
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Set, Tuple

import torch


class AccelerationPluginConfigError(Exception):
    """A plugin found its configuration section but a key or value in it is invalid."""


@dataclass
class PluginRegistration:
    plugin: type
    AND: Optional[List[str]] = None
    OR: Optional[List[str]] = None
    package_name: Optional[str] = None
    package_version: Optional[str] = None


PLUGIN_REGISTRATIONS: List[PluginRegistration] = []

_MISSING = object()


def _trace_key_path(configuration: Dict, key: str):
    """Follow a dotted key path through nested dicts; ``None`` when any component is absent."""
    node: Any = configuration
    for part in key.split("."):
        if not isinstance(node, dict) or part not in node:
            return None
        node = node[part]
    return node


def _graft(tree: Dict, dotted: str, content: Any) -> None:
    parts = dotted.split(".")
    for part in parts[:-1]:
        tree = tree.setdefault(part, {})
    tree[parts[-1]] = content


def get_relevant_configuration_sections(configuration: Dict) -> List[Tuple[Dict, type]]:
    selected: List[Tuple[Dict, type]] = []
    for reg in PLUGIN_REGISTRATIONS:
        and_paths = reg.AND or []
        or_paths = reg.OR or []
        section: Dict = {}

        and_hits = [(p, _trace_key_path(configuration, p)) for p in and_paths]
        and_ok = all(v is not None for _, v in and_hits)
        if and_ok:
            for p, v in and_hits:
                _graft(section, p, v)
        or_hits = [(p, _trace_key_path(configuration, p)) for p in or_paths]
        or_hits = [(p, v) for p, v in or_hits if v is not None]
        for p, v in or_hits:
            _graft(section, p, v)

        # rejected when an AND path is missing and no OR path rescued it
        if not and_ok and not or_hits:
            continue
        if section:
            selected.append((section, reg.plugin))
    return selected


class AccelerationPlugin:
    """Base class of all acceleration plugins.

    Lifecycle hooks (all optional): ``model_loader`` (when ``requires_custom_loading``), ``augmentation``
    (when ``requires_augmentation``) and ``get_callbacks_and_ready_for_train``.
    """

    # when set, the model must declare at least one of these architectures
    restricted_model_archs: Optional[Set[str]] = None
    # importable packages the plugin cannot work without
    require_packages: Optional[Set[str]] = None

    @staticmethod
    def register_plugin(
        plugin: type,
        configuration_and_paths: Optional[List[str]] = None,
        configuration_or_paths: Optional[List[str]] = None,
        **kwargs,
    ) -> None:
        assert (configuration_and_paths is not None and len(configuration_and_paths) > 0) or (
            configuration_or_paths is not None and len(configuration_or_paths) > 0
        ), "Specify at least one AND or OR path"

        module = sys.modules.get(plugin.__module__)
        pkg_name = getattr(module, "__package__", None)
        pkg_version = None
        if pkg_name:
            try:
                pkg_version = importlib.metadata.version(pkg_name.split(".")[0])
            except importlib.metadata.PackageNotFoundError:
                try:
                    from .. import __version__ as pkg_version  # in-tree plugins share the framework version
                except Exception:  # pragma: no cover
                    pkg_version = None
        PLUGIN_REGISTRATIONS.append(
            PluginRegistration(
                plugin=plugin,
                AND=configuration_and_paths,
                OR=configuration_or_paths,
                package_name=pkg_name,
                package_version=pkg_version,
            )
        )

    def __init__(self, configurations: Dict[str, Dict]):
        self.configurations = configurations

    @property
    def requires_custom_loading(self) -> bool:
        return False

    @property
    def requires_augmentation(self) -> bool:
        return False

    def model_loader(self, model_name: str, **kwargs):
        raise NotImplementedError

    def augmentation(self, model: torch.nn.Module, train_args, modifiable_args: Tuple):
        raise NotImplementedError

    def get_callbacks_and_ready_for_train(self, model: torch.nn.Module = None, accelerator=None):
        return []

    # ------------------------------------------------------------------ configuration validators
    def _check_config_and_maybe_check_values(self, key: str, values: Optional[List[Any]] = None, default: Any = None):
        found = _trace_key_path(self.configurations, key)
        name = self.__class__.__name__

        if values is None:
            if found is None:
                if default is None:
                    raise AccelerationPluginConfigError(f"{name}: '{key}' was not a valid configuration config")
                return default
            return found

        if isinstance(found, dict):
            if len(found) > 1:
                raise AccelerationPluginConfigError(
                    f"{name}: '{key}' found but amongst multiple '{list(found.keys())}' exist. "
                    f"Ambiguous check in expected set '{values}'."
                )
            found = next(iter(found.keys()))

        if found in values:
            return found
        if found is None and default is not None:
            return default
        raise AccelerationPluginConfigError(
            f"{name}: Value at '{key}' was '{found}'. Not found in expected set '{values}'."
        )

    def _check_config_equal(self, key: str, value: Any, **kwargs):
        return self._check_config_and_maybe_check_values(key, [value], **kwargs)
