"""Registries for datasets, processors and models plus model construction.

Same decorator surface as the reference (src/lmms_engine/mapping_func.py:13-159):
``@register_dataset(name)``, ``@register_processor(name)``,
``register_model(model_type, ConfigCls, ModelCls, model_general_type)``,
``create_model_from_pretrained`` / ``create_model_from_config``.  Native model classes are
resolved from ``config.json``'s ``model_type``; when no native class is registered and
``transformers`` is importable the HF Auto classes are used as a fallback so every family
the reference can load still loads.
"""
from __future__ import annotations

import json
import os
from typing import Any, Callable, Dict, Optional, Tuple, Type

DATASET_MAPPING: Dict[str, type] = {}
DATAPROCESSOR_MAPPING: Dict[str, type] = {}
# model_type -> {general_type: (ConfigCls, ModelCls)}
MODEL_REGISTRY: Dict[str, Dict[str, Tuple[type, type]]] = {}
AUTO_REGISTER_MODEL_MAPPING = ("causal_lm", "masked_lm", "image_text_to_text", "general")


def register_dataset(name: str) -> Callable[[type], type]:
    def deco(cls):
        DATASET_MAPPING[name] = cls
        return cls

    return deco


def register_processor(name: str) -> Callable[[type], type]:
    def deco(cls):
        DATAPROCESSOR_MAPPING[name] = cls
        return cls

    return deco


def register_model(model_type: str, config_cls: type, model_cls: type, model_general_type: str = "causal_lm") -> None:
    if model_general_type not in AUTO_REGISTER_MODEL_MAPPING:
        raise ValueError(f"model_general_type must be one of {AUTO_REGISTER_MODEL_MAPPING}")
    MODEL_REGISTRY.setdefault(model_type, {})[model_general_type] = (config_cls, model_cls)


def _resolve(model_type: str, general_type: Optional[str]):
    entry = MODEL_REGISTRY.get(model_type)
    if not entry:
        return None
    if general_type is not None:
        if general_type not in entry:
            raise KeyError(f"{model_type} is not registered as {general_type}; have {list(entry)}")
        return entry[general_type]
    for key in ("image_text_to_text", "causal_lm", "masked_lm", "general"):
        if key in entry:
            return entry[key]
    return None


def create_model_from_config(model_type: str, config: Dict[str, Any], model_general_type: Optional[str] = None,
                             device=None, dtype=None, **kw):
    """Random-init model from a config dict (``model_config.load_from_config``).  With
    ``device`` / ``dtype`` the parameters are created (and initialised) directly there, so a
    multi-billion-parameter model never takes a detour through fp32 host memory."""
    import torch

    from . import models  # noqa: F401  (populates the registry)

    hit = _resolve(model_type, model_general_type)
    if hit is not None:
        cfg_cls, model_cls = hit
        cfg = cfg_cls.from_dict({"model_type": model_type, **(config or {})})
        if device is None and dtype is None:
            return model_cls(cfg)
        old = torch.get_default_dtype()
        try:
            if dtype is not None:
                torch.set_default_dtype(dtype)
            with torch.device(device if device is not None else "cpu"):
                return model_cls(cfg)
        finally:
            torch.set_default_dtype(old)
    return _hf_fallback_from_config(model_type, config, model_general_type, **kw)


def create_model_from_pretrained(path: str, model_general_type: Optional[str] = None, **kw):
    """Model + weights from an HF-style directory (``config.json`` + safetensors)."""
    from . import models  # noqa: F401
    from .models import hf_io

    cfg_path = os.path.join(path, "config.json")
    if os.path.exists(cfg_path):
        with open(cfg_path) as f:
            raw = json.load(f)
        hit = _resolve(raw.get("model_type", ""), model_general_type)
        if hit is not None:
            cfg_cls, model_cls = hit
            model = model_cls(cfg_cls.from_dict(raw))
            hf_io.load_pretrained_weights(model, path)
            return model
    return _hf_fallback_from_pretrained(path, model_general_type, **kw)


def _hf_auto_class(general_type: Optional[str]):
    import transformers

    return {
        None: transformers.AutoModelForCausalLM,
        "causal_lm": transformers.AutoModelForCausalLM,
        "masked_lm": transformers.AutoModelForMaskedLM,
        "image_text_to_text": getattr(transformers, "AutoModelForImageTextToText", transformers.AutoModel),
        "general": transformers.AutoModel,
    }[general_type]


def _hf_fallback_from_config(model_type, config, general_type, **kw):
    import transformers

    cfg = transformers.AutoConfig.for_model(model_type, **(config or {}))
    return _hf_auto_class(general_type).from_config(cfg, **kw)


def _hf_fallback_from_pretrained(path, general_type, **kw):
    return _hf_auto_class(general_type).from_pretrained(path, **kw)
