"""Registry of per-model parallel plans (TP / EP + FSDP2)
(reference: src/lmms_engine/parallel/parallelize.py:1-39)."""
from __future__ import annotations

from typing import Callable, Dict

MODEL_TO_PARALLEL_METHOD: Dict[str, Callable] = {}


def register_parallel_plan(model_type: str):
    def deco(fn):
        MODEL_TO_PARALLEL_METHOD[model_type] = fn
        return fn

    return deco


def has_parallel_plan(model_type) -> bool:
    _load_plans()
    return model_type in MODEL_TO_PARALLEL_METHOD


def apply_parallelize(model, model_type: str, train_args, dtype=None, **kwargs):
    _load_plans()
    if model_type not in MODEL_TO_PARALLEL_METHOD:
        raise KeyError(f"no parallel plan registered for model_type '{model_type}'")
    return MODEL_TO_PARALLEL_METHOD[model_type](model, train_args, dtype=dtype, **kwargs)


_loaded = False


def _load_plans():
    global _loaded
    if _loaded:
        return
    _loaded = True
    try:
        from . import plans  # noqa: F401
    except ImportError:
        pass
