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


def native_kernels_apply(family: str) -> Callable:
    """What ``apply_liger_kernel_to_<family>`` is here.  The reference swaps library modules for Liger / unpadded ones
    with these functions (src/lmms_engine/models/<family>/monkey_patch.py); the native models run the fused kernels
    from the start, so the function has nothing to swap: it accepts the reference's arguments and runs the patches a
    user registered for the family, if a model is given."""

    def apply(model=None, **kwargs) -> int:
        return MONKEY_PATCHER.apply(model, family, ["liger"], **kwargs) if model is not None else 0

    apply.__name__ = f"apply_liger_kernel_to_{family}"
    apply.__doc__ = native_kernels_apply.__doc__
    return apply
