"""Attention and distributed packing: padding-free batches and the multipack sampler."""
from .framework_plugin_padding_free import PaddingFreeAccelerationPlugin  # noqa: F401
from .framework_plugin_multipack import MultipackDataloaderAccelerationPlugin  # noqa: F401
