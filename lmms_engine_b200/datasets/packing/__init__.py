"""Sequence packing strategies (online/streaming and offline), backed by the C++ core in
``csrc/host/packing.cpp``.  Registry and names follow the reference
(src/lmms_engine/datasets/packing/__init__.py:10-28)."""
from .base import OnlinePackingStrategy
from .online import (BalancedPacking, BestFitPacking, FirstFitPacking, TrueFirstFitPacking, build_online_packer,
                     ONLINE_PACKERS)
from .offline import pack_by_first_fit, pack_by_window, build_offline_groups

__all__ = [
    "OnlinePackingStrategy", "FirstFitPacking", "BestFitPacking", "BalancedPacking", "TrueFirstFitPacking",
    "build_online_packer", "ONLINE_PACKERS", "pack_by_first_fit", "pack_by_window", "build_offline_groups",
]
