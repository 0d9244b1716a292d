"""Processors: chat rendering, label masking, image / video patchification."""
from . import chat  # noqa: F401  (registers the processors)
from . import llava_ov2_processor  # noqa: F401
from . import generative_processors  # noqa: F401
from .chat import ChatProcessor, Qwen3VLProcessor, QwenVLProcessor
from .tokenizer import ByteChatTokenizer, load_tokenizer

__all__ = ["ChatProcessor", "QwenVLProcessor", "Qwen3VLProcessor", "ByteChatTokenizer", "load_tokenizer"]
