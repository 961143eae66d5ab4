"""Helpers for testing plugins and patchers in isolation.

Same helper names and behaviour as fms_acceleration/utils/test_utils.py:32-228 of the reference: the
context managers snapshot the process-wide registries (plugin registrations, the framework's class-level
active lists, the two patcher singletons), install fresh ones for the duration of the ``with`` block and
restore the snapshot afterwards, also when the body raises.
"""
from __future__ import annotations

import os
import tempfile
from contextlib import contextmanager
from typing import Any, Callable, Dict, List, Optional, Set

import torch
import yaml

from ..constants import KEY_PLUGINS
from ..framework import AccelerationFramework
from ..framework_plugin import PLUGIN_REGISTRATIONS, AccelerationPlugin


def update_configuration_contents(configuration_contents: Dict, augment_at_path: str, augmented_contents: Any) -> Dict:
    """Edit a nested config: if the node at ``augment_at_path`` is a dict, RENAME its key to
    ``augmented_contents``; otherwise replace its value."""
    *parents, leaf = augment_at_path.split(".")
    node = configuration_contents
    for k in parents:
        node = node[k]
    if isinstance(node[leaf], dict):
        node[augmented_contents] = node.pop(leaf)
    else:
        node[leaf] = augmented_contents
    return configuration_contents


def read_configuration(path: str) -> Dict:
    with open(path, encoding="utf-8") as fh:
        return yaml.safe_load(fh)


def configure_framework_from_json(configuration_contents: Dict, require_packages_check: bool = True):
    fd, name = tempfile.mkstemp(suffix=".yaml")
    try:
        with os.fdopen(fd, "w", encoding="utf-8") as fh:
            yaml.dump({KEY_PLUGINS: configuration_contents}, fh)
        return AccelerationFramework(name, require_packages_check)
    finally:
        os.unlink(name)


@contextmanager
def build_framework_and_maybe_instantiate(
    plugins_to_be_registered: List[tuple],
    configuration_contents: Optional[Dict] = None,
    instantiate: bool = True,
    reset_registrations: bool = True,
    require_packages_check: bool = True,
):
    """Register ``(and_paths, plugin)`` or ``(and_paths, or_paths, plugin)`` entries and (optionally) yield an
    ``AccelerationFramework`` built from ``configuration_contents``."""
    configuration_contents = configuration_contents or {}
    saved_regs = list(PLUGIN_REGISTRATIONS)
    saved_active = AccelerationFramework.active_plugins
    saved_loaders = AccelerationFramework.plugins_require_custom_loading
    if reset_registrations:
        PLUGIN_REGISTRATIONS.clear()
    AccelerationFramework.active_plugins = []
    AccelerationFramework.plugins_require_custom_loading = []
    try:
        for entry in plugins_to_be_registered:
            if len(entry) == 2:
                and_paths, plugin = entry
                or_paths = None
            else:
                and_paths, or_paths, plugin = entry
            AccelerationPlugin.register_plugin(
                plugin, configuration_and_paths=and_paths, configuration_or_paths=or_paths
            )
        if instantiate:
            yield configure_framework_from_json(configuration_contents, require_packages_check)
        else:
            yield
    finally:
        if reset_registrations:
            PLUGIN_REGISTRATIONS.clear()
            PLUGIN_REGISTRATIONS.extend(saved_regs)
        AccelerationFramework.active_plugins = saved_active
        AccelerationFramework.plugins_require_custom_loading = saved_loaders


build_framework_and_instantiate = build_framework_and_maybe_instantiate


def instantiate_framework(configuration_contents: Dict, require_packages_check: bool = True):
    """As above but keeps the current plugin registrations (uses the really imported plugins)."""
    return build_framework_and_instantiate(
        [], configuration_contents, reset_registrations=False, require_packages_check=require_packages_check
    )


def create_noop_model_with_archs(class_name: str = "ModelNoop", archs: Optional[List[str]] = None):
    config = type("Config", (object,), {"architectures": archs or []})
    return type(class_name, (torch.nn.Module,), {"config": config})


def create_plugin_cls(
    class_name: str = "PluginNoop",
    restricted_models: Optional[Set] = None,
    require_pkgs: Optional[Set] = None,
    requires_custom_loading: bool = False,
    requires_augmentation: bool = False,
    augmentation: Optional[Callable] = None,
    model_loader: Optional[Callable] = None,
):
    attrs = {
        "restricted_model_archs": restricted_models or set(),
        "require_packages": require_pkgs or set(),
        "requires_custom_loading": requires_custom_loading,
        "requires_augmentation": requires_augmentation,
    }
    if augmentation is not None:
        attrs["augmentation"] = augmentation
    if model_loader is not None:
        attrs["model_loader"] = model_loader
    return type(class_name, (AccelerationPlugin,), attrs)


def dummy_augmentation(self, model, train_args, modifiable_args):
    return model, modifiable_args


def dummy_custom_loader(self, model_name, **kwargs):
    return create_noop_model_with_archs(archs=["DummyModel"])


@contextmanager
def instantiate_model_patcher():
    from collections import OrderedDict

    from ..model_patcher import ModelPatcher

    saved_rules, saved_history = ModelPatcher.rules, ModelPatcher.history
    ModelPatcher.rules, ModelPatcher.history = OrderedDict(), []
    try:
        yield
    finally:
        ModelPatcher.rules, ModelPatcher.history = saved_rules, saved_history


@contextmanager
def instantiate_accel_patcher():
    from ..accelerator_patcher import AcceleratorPatcher

    saved_rules, saved_history = AcceleratorPatcher.replacement_rules, AcceleratorPatcher.history
    AcceleratorPatcher.replacement_rules, AcceleratorPatcher.history = {}, []
    try:
        yield
    finally:
        AcceleratorPatcher.replacement_rules, AcceleratorPatcher.history = saved_rules, saved_history
