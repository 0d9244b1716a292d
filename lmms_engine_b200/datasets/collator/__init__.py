from .packed_collator import PackedCollator
from .vision_collator import VisionCollator

__all__ = ["PackedCollator", "VisionCollator"]
