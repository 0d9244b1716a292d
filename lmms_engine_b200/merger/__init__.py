from .base import CheckpointMerger
from .consolidate import consolidate, consolidate_key

__all__ = ["CheckpointMerger", "FSDP2Merger", "consolidate", "consolidate_key"]


def __getattr__(name):
    if name == "FSDP2Merger":
        from .fsdp2 import FSDP2Merger

        return FSDP2Merger
    raise AttributeError(name)
