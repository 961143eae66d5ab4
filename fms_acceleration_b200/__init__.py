"""B200-native fine-tuning acceleration framework (sm_100a kernels + PyTorch framework layer)."""

__version__ = "0.1.0"
