"""B200-native multimodal training engine (sm_100a kernels + PyTorch orchestration)."""
__version__ = "0.1.0"
