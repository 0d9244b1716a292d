"""Merger interface (reference: src/lmms_engine/merger/base.py:1-26)."""
from abc import ABC, abstractmethod
from pathlib import Path
from typing import Optional


class CheckpointMerger(ABC):
    def __init__(self, checkpoint_path: str, output_path: Optional[str] = None):
        self.checkpoint_path = Path(checkpoint_path)
        self.output_path = Path(output_path) if output_path else None

    @abstractmethod
    def merge(self) -> Path: ...
