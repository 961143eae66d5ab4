"""Helpers shipped with the framework: the testing utilities are importable from the package itself
(``from fms_acceleration.utils import instantiate_framework, read_configuration``), as in the reference
(fms_acceleration/utils/__init__.py:16)."""
from .test_utils import (build_framework_and_maybe_instantiate, configure_framework_from_json, create_noop_model_with_archs,
                         create_plugin_cls, dummy_augmentation, dummy_custom_loader, instantiate_accel_patcher,
                         instantiate_framework, instantiate_model_patcher, read_configuration,
                         update_configuration_contents)

__all__ = ["build_framework_and_maybe_instantiate", "configure_framework_from_json", "create_noop_model_with_archs",
           "create_plugin_cls", "dummy_augmentation", "dummy_custom_loader", "instantiate_accel_patcher",
           "instantiate_framework", "instantiate_model_patcher", "read_configuration", "update_configuration_contents"]
