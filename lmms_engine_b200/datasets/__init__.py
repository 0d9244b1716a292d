"""Data plane: dataset / processor registries, packing, collators."""
from .config import DatasetConfig, ProcessorConfig

__all__ = ["DatasetConfig", "ProcessorConfig"]
