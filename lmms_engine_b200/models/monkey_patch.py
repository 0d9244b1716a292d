"""Extension point for model patches (reference: src/lmms_engine/models/monkey_patch.py and the
``@MONKEY_PATCHER.register(model_type, patch_type)`` decorators of every model family).

The native models need no patching: varlen packing, fused kernels and sequence parallelism are
part of their forward pass.  The registry is kept so that user code written against the reference
can still hook a model type: a registered function is called as ``fn(model, **monkey_patch_kwargs)``
by the runner after the model is built, for every ``patch_type`` the config asks for
(``monkey_patch_kwargs.patch_type``, default ``["liger"]``).
"""
from __future__ import annotations

from typing import Callable, Dict, List, Tuple


class MonkeyPatcher:
    def __init__(self):
        self._patches: Dict[Tuple[str, str], List[Callable]] = {}

    def register(self, model_type: str, patch_type: str = "liger"):
        def deco(fn: Callable):
            self._patches.setdefault((model_type, patch_type), []).append(fn)
            return fn

        return deco

    def registered(self, model_type: str, patch_type: str) -> List[Callable]:
        return list(self._patches.get((model_type, patch_type), []))

    def apply(self, model, model_type: str, patch_types, **kwargs) -> int:
        """Run every patch registered for ``model_type``; returns how many ran."""
        if isinstance(patch_types, str):
            patch_types = [patch_types]
        n = 0
        for pt in patch_types or []:
            for fn in self.registered(model_type, pt):
                fn(model, **kwargs)
                n += 1
        return n


MONKEY_PATCHER = MonkeyPatcher()
