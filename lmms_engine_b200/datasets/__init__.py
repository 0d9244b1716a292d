"""Data plane: dataset / processor registries, packing, collators."""
from .config import DatasetConfig, ProcessorConfig

__all__ = ["DatasetConfig", "ProcessorConfig"]

from ._public_names import exported as _exported

__getattr__ = _exported(['MultiModalDataset', 'VisionSFTDataset', 'VisionAudioSFTDataset', 'FinewebEduDataset', 'MultiModalIterableDataset', 'VisionSFTIterableDataset'])
