"""Processors: chat rendering, label masking, image / video patchification."""
from . import chat  # noqa: F401  (registers the processors)
from . import llava_ov2_processor  # noqa: F401
from . import generative_processors  # noqa: F401
from ..config import ProcessorConfig  # noqa: F401
from .chat import ChatProcessor, Qwen3VLProcessor, QwenVLProcessor
from .tokenizer import ByteChatTokenizer, load_tokenizer

__all__ = ["ChatProcessor", "QwenVLProcessor", "Qwen3VLProcessor", "ByteChatTokenizer", "load_tokenizer"]

from .._public_names import exported as _exported

__getattr__ = _exported(['AeroDataProcessor', 'AeroRealtimeDataProcessor', 'BagelDataProcessor', 'BaseQwen2_5_DataProcessor', 'LLaVADataProcessor', 'LLaVAVideoDataProcessor', 'LlavaOnevision2DataProcessor', 'NanovlmDataProcessor', 'PureTextDataProcessor', 'Qwen2DataProcessor', 'Qwen2VLDataProcessor', 'Qwen2_5OmniDataProcessor', 'Qwen2_5_VLDataProcessor', 'Qwen3OmniMoeDataProcessor', 'Qwen3_VLDataProcessor', 'RaeSiglipDataProcessor', 'SitDataProcessor', 'WanVideoDataProcessor'])
