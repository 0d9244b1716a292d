"""Utilities.  The five names the reference exports here (src/lmms_engine/utils/__init__.py) resolve on first use, so
that importing a light helper does not import torch-heavy modules."""
import importlib

_EXPORTS = {"ComputeTracker": "compute_tracker", "DataUtilities": "data_utils", "Logging": "logging_utils", "StepProfiler": "profiler",
            "TrainUtilities": "train_utils"}
__all__ = sorted(_EXPORTS)


def __getattr__(name):
    if name in _EXPORTS:
        return getattr(importlib.import_module(f"{__name__}.{_EXPORTS[name]}"), name)
    raise AttributeError(name)
