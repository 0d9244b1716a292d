from .multimodal_dataset import MultiModalDataset  # noqa: F401

from .._public_names import exported as _exported

__getattr__ = _exported(['BaseDataset', 'VisionSFTDataset', 'VisionAudioSFTDataset', 'QwenOmniSFTDataset', 'Qwen3VLDataset', 'RaeDataset', 'SitDataset', 'LLaVAVideoDataset'])
