"""Streaming packer interface (reference: src/lmms_engine/datasets/packing/base.py:16-56)."""
from abc import ABC, abstractmethod
from typing import Any, Iterator, List


class OnlinePackingStrategy(ABC):
    """``for item, n in stream: yield from packer.add(item, n)`` then ``yield from packer.flush()``.

    Every yielded pack is a list of items whose lengths sum to at most ``packing_length``.
    Samples longer than ``packing_length`` must be handled by the caller.
    """

    def __init__(self, packing_length: int) -> None:
        self.packing_length = packing_length

    @abstractmethod
    def add(self, item: Any, length: int) -> Iterator[List[Any]]: ...

    @abstractmethod
    def flush(self) -> Iterator[List[Any]]: ...
