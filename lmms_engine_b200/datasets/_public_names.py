"""The class names under which the reference exports its datasets, processors and collators
(src/lmms_engine/datasets/{__init__,naive/__init__,iterable/__init__,collator/__init__,processor/__init__}.py), resolved
to this package's classes: a dataset or processor by the name it is registered under, a collator or base class by
module and attribute.  Code written against the reference (``from lmms_engine.datasets.naive import VisionSFTDataset``,
a subclass of ``BaseDataset`` registered with ``@register_dataset``) keeps importing."""
from __future__ import annotations

import importlib

DATASETS = {
    "VisionSFTDataset": "vision", "VisionAudioSFTDataset": "vision_audio", "QwenOmniSFTDataset": "qwen_omni",
    "Qwen3VLDataset": "qwen3_vl", "RaeDataset": "rae", "SitDataset": "sit", "LLaVAVideoDataset": "llava_video",
    "VisionSFTIterableDataset": "vision_iterable", "AeroRealtimeIterableDataset": "aero_realtime_iterable",
    "BagelIterableDataset": "bagel_iterable", "FinewebEduDataset": "fineweb_edu", "LlavaOv2IterableDataset": "llava_ov2_iterable",
    "Qwen3VLIterableDataset": "qwen3_vl_iterable", "QwenOmniIterableDataset": "qwen_omni_iterable",
}
PROCESSORS = {
    "AeroDataProcessor": "aero", "AeroRealtimeDataProcessor": "aero_realtime", "BagelDataProcessor": "bagel",
    "BaseQwen2_5_DataProcessor": "qwen2_5_vl", "LlavaOnevision2DataProcessor": "llava_onevision2", "LLaVADataProcessor": "llava",
    "LLaVAVideoDataProcessor": "llava_video", "NanovlmDataProcessor": "nanovlm", "PureTextDataProcessor": "pure_text",
    "Qwen2_5OmniDataProcessor": "Qwen2_5OmniProcessor", "Qwen2_5_VLDataProcessor": "qwen2_5_vl", "Qwen2DataProcessor": "qwen2",
    "Qwen2VLDataProcessor": "qwen2_vl", "Qwen3OmniMoeDataProcessor": "Qwen3OmniMoeProcessor", "Qwen3_VLDataProcessor": "qwen3_vl",
    "RaeSiglipDataProcessor": "rae_siglip", "SitDataProcessor": "sit", "WanVideoDataProcessor": "wanvideo",
}
ATTRIBUTES = {
    "BaseDataset": ("naive.multimodal_dataset", "MultiModalDataset"),
    "MultiModalDataset": ("naive.multimodal_dataset", "MultiModalDataset"),
    "BaseIterableDataset": ("iterable.multimodal_iterable_dataset", "MultiModalIterableDataset"),
    "MultiModalIterableDataset": ("iterable.multimodal_iterable_dataset", "MultiModalIterableDataset"),
    "VisionCollator": ("collator.vision_collator", "VisionCollator"),
    "LLaVACollator": ("collator.vision_collator", "LLaVACollator"),
    "BagelCollator": ("extra", "BagelCollator"),
    "AeroRealtimeCollator": ("realtime", "RealtimeCollator"),
}


def resolve(name: str):
    """The class exported as ``name``; ``AttributeError`` for a name the reference does not export either."""
    if name in ATTRIBUTES:
        module, attr = ATTRIBUTES[name]
        return getattr(importlib.import_module(f"{__package__}.{module}"), attr)
    if name in DATASETS or name in PROCESSORS:
        from .. import mapping_func
        from . import registry  # noqa: F401  (fills both tables)

        table, key = (mapping_func.DATASET_MAPPING, DATASETS[name]) if name in DATASETS else (mapping_func.DATAPROCESSOR_MAPPING, PROCESSORS[name])
        return table[key]
    raise AttributeError(name)


def exported(names):
    """A module-level ``__getattr__`` that answers for ``names`` only."""
    names = frozenset(names)

    def __getattr__(name):
        if name in names:
            return resolve(name)
        raise AttributeError(name)

    return __getattr__
