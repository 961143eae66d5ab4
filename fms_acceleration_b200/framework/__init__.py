"""Framework core: plugin registry, ``AccelerationFramework`` and the two patcher singletons."""
from .constants import ACCELERATION_FRAMEWORK_ENV_KEY, KEY_PLUGINS, PLUGIN_PREFIX, PLUGINS
from .framework import AccelerationFramework
from .framework_plugin import (
    PLUGIN_REGISTRATIONS,
    AccelerationPlugin,
    AccelerationPluginConfigError,
    get_relevant_configuration_sections,
)

__all__ = [
    "AccelerationFramework",
    "AccelerationPlugin",
    "AccelerationPluginConfigError",
    "get_relevant_configuration_sections",
    "PLUGIN_REGISTRATIONS",
    "KEY_PLUGINS",
    "PLUGINS",
    "PLUGIN_PREFIX",
    "ACCELERATION_FRAMEWORK_ENV_KEY",
]
