"""Structural protocols (reference: src/lmms_engine/protocol/lmms_proto.py:1-14)."""
from typing import Protocol, runtime_checkable


@runtime_checkable
class Runnable(Protocol):
    def build(self): ...

    def run(self, **kwargs): ...


@runtime_checkable
class Processable(Protocol):
    def build(self): ...

    def process(self, *args, **kwargs): ...
