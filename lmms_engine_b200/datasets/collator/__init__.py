from .packed_collator import PackedCollator
from .vision_collator import VisionCollator

__all__ = ["PackedCollator", "VisionCollator"]

from .._public_names import exported as _exported

__getattr__ = _exported(['AeroRealtimeCollator', 'BagelCollator', 'LLaVACollator'])
