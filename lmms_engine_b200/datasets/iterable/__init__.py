from .multimodal_iterable_dataset import MultiModalIterableDataset  # noqa: F401

from .._public_names import exported as _exported

__getattr__ = _exported(['AeroRealtimeIterableDataset', 'BaseIterableDataset', 'FinewebEduDataset', 'VisionSFTIterableDataset', 'BagelIterableDataset', 'LlavaOv2IterableDataset', 'Qwen3VLIterableDataset', 'QwenOmniIterableDataset'])
