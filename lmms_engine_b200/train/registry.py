"""Trainer registry (reference: src/lmms_engine/train/registry.py:1-42)."""
from typing import Callable, Dict, Iterator


class TrainerRegister:
    def __init__(self) -> None:
        self._trainers: Dict[str, type] = {}

    def register(self, name: str) -> Callable[[type], type]:
        def deco(cls):
            self._trainers[name] = cls
            return cls

        return deco

    def __getitem__(self, name: str) -> type:
        if name not in self._trainers:
            raise KeyError(f"trainer '{name}' is not registered; known: {sorted(self._trainers)}")
        return self._trainers[name]

    def __contains__(self, name: str) -> bool:
        return name in self._trainers

    def __iter__(self) -> Iterator[str]:
        return iter(self._trainers)

    def keys(self):
        return self._trainers.keys()

    def get(self, name, default=None):
        return self._trainers.get(name, default)


TRAINER_REGISTER = TrainerRegister()
