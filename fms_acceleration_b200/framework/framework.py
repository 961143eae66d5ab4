"""``AccelerationFramework``: reads the acceleration YAML, activates plugins, dispatches the lifecycle.

Contract of fms_acceleration/framework.py:85-261 in the reference: the YAML must have a top-level
``plugins`` mapping; each registered plugin whose key paths match is instantiated with its sub-config;
missing ``require_packages`` is an error unless ``require_packages_check=False``; at most one active plugin
may load the model; ``augmentation`` enforces ``restricted_model_archs``; ``get_callbacks_and_ready_for_train``
applies the ModelPatcher and AcceleratorPatcher rules and returns the plugins' trainer callbacks.
"""
from __future__ import annotations

import importlib.util
import logging
import os
from typing import Callable, List, Optional, Set, Tuple

import torch
import yaml

from .constants import ACCELERATION_FRAMEWORK_ENV_KEY, KEY_PLUGINS
from .framework_plugin import (
    PLUGIN_REGISTRATIONS,
    AccelerationPlugin,
    PluginRegistration,
    get_relevant_configuration_sections,
)

logger = logging.getLogger(__name__)


def _is_package_available(name: str) -> bool:
    try:
        return importlib.util.find_spec(name) is not None
    except (ImportError, ValueError):
        return False


def log_patch_summary(summary: List[str], logging_func: Optional[Callable] = None) -> None:
    emit = logging_func or print
    for line in summary:
        emit(line)


def check_plugin_packages(plugin: AccelerationPlugin):
    if plugin.require_packages is None:
        return True, []
    missing = [p for p in plugin.require_packages if not _is_package_available(p)]
    return len(missing) == 0, missing


def log_initialization_message(
    active_class_names: Set[str],
    registered_plugins: List[PluginRegistration],
    logging_func: Optional[Callable] = None,
) -> None:
    emit = logging_func or print
    emit("***** FMS AccelerationFramework *****")
    for reg in registered_plugins:
        if reg.plugin.__name__ in active_class_names:
            emit(
                f"Active Plugin: {reg.plugin.__name__}. "
                f"Python package: {reg.package_name}. "
                f"Version: {reg.package_version}."
            )


def read_configuration_file(configuration_file: str) -> dict:
    with open(configuration_file, "r", encoding="utf-8") as fh:
        contents = yaml.safe_load(fh)
    if not isinstance(contents, dict) or contents.get(KEY_PLUGINS) is None:
        raise ValueError(f"Configuration file must contain a '{KEY_PLUGINS}' body")
    return dict(contents[KEY_PLUGINS].items())


class AccelerationFramework:
    # Class-level state, as in the reference (framework.py:97-98): a second instance created in the same
    # process sees the plugins of the first.  The test helpers snapshot and restore these lists.
    active_plugins: List[Tuple[str, AccelerationPlugin]] = []
    plugins_require_custom_loading: List[str] = []

    @classmethod
    def reset(cls) -> None:
        """Forget the plugins activated by an earlier instance.  The active lists are class-level (one framework per
        process, as in the reference); a process that configures a second framework calls this first."""
        cls.active_plugins = []
        cls.plugins_require_custom_loading = []

    def __init__(self, configuration_file: Optional[str] = None, require_packages_check: bool = True):
        env_file = os.environ.get(ACCELERATION_FRAMEWORK_ENV_KEY)
        if configuration_file is None and env_file is None:
            raise ValueError(
                "configuration_file is not passed into configuration_file but "
                f"{ACCELERATION_FRAMEWORK_ENV_KEY} is not set. Please choose one "
                "of the means to initialize the framework."
            )

        plugin_configs: dict = {}
        if configuration_file is not None:
            plugin_configs = read_configuration_file(configuration_file)
        if env_file is not None and (configuration_file is None or len(plugin_configs) == 0):
            plugin_configs = read_configuration_file(env_file)

        for section, cls in get_relevant_configuration_sections(plugin_configs):
            plugin_name = str(cls.__name__)
            plugin = cls(section)

            ok, missing = check_plugin_packages(plugin)
            if not ok and require_packages_check:
                raise ValueError(
                    f"Packages '{', '.join(missing)}' required by activated plugin '{plugin_name}' "
                    "is missing. Please install it."
                )
            if any(name == plugin_name for name, _ in self.active_plugins):
                continue  # one instance per plugin class
            self.active_plugins.append((plugin_name, plugin))
            if plugin.requires_custom_loading:
                self.plugins_require_custom_loading.append(plugin_name)

        if len(self.active_plugins) == 0:
            raise ValueError(
                "No plugins could be configured. Please check the acceleration "
                "framework configuration file."
            )
        assert len(self.plugins_require_custom_loading) <= 1, (
            "Can load at most 1 plugin with custom model loading, "
            f"but tried to '{self.plugins_require_custom_loading}'."
        )

    # ------------------------------------------------------------------ lifecycle
    def model_loader(self, model_name: str, **kwargs):
        if len(self.plugins_require_custom_loading) == 0:
            raise NotImplementedError(
                "Attempted model loading, but none "
                f"of activated plugins '{list(self.active_plugins)}' "
                "require custom loading."
            )
        wanted = self.plugins_require_custom_loading[0]
        plugin = next(p for name, p in self.active_plugins if name == wanted)
        return plugin.model_loader(model_name, **kwargs)

    def augmentation(self, model, train_args, modifiable_args: Tuple):
        # a model without a ``config`` is an error (AttributeError), as in the reference; a config that lists no
        # architectures matches no restricted plugin
        archs = getattr(model.config, "architectures", None)
        model_archs = set(archs if archs is not None else [])
        for plugin_name, plugin in self.active_plugins:
            if plugin.restricted_model_archs and not any(a in model_archs for a in plugin.restricted_model_archs):
                raise ValueError(
                    f"Model architectures in '{model_archs}' are not supported for '{plugin_name}'."
                )
            if plugin.requires_augmentation:
                model, modifiable_args = plugin.augmentation(model, train_args, modifiable_args=modifiable_args)
        return model, modifiable_args

    @property
    def requires_custom_loading(self) -> bool:
        return len(self.plugins_require_custom_loading) > 0

    @property
    def requires_augmentation(self) -> bool:
        return any(p.requires_augmentation for _, p in self.active_plugins)

    def get_callbacks_and_ready_for_train(self, model: torch.nn.Module = None, accelerator=None):
        from .accelerator_patcher import AcceleratorPatcher
        from .model_patcher import ModelPatcher

        if model is not None:
            ModelPatcher.patch(model)
        if accelerator is not None:
            AcceleratorPatcher.patch(accelerator)

        if accelerator is not None and getattr(accelerator, "is_main_process", True):
            log_initialization_message({n for n, _ in self.active_plugins}, PLUGIN_REGISTRATIONS, logger.info)
            log_patch_summary(ModelPatcher.summary(raw=False).split("\n"), logger.info)
            log_patch_summary(AcceleratorPatcher.summary().split("\n"), logger.info)

        callbacks = []
        for _, plugin in self.active_plugins:
            callbacks.extend(plugin.get_callbacks_and_ready_for_train(model, accelerator))
        return callbacks
