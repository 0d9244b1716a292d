"""Dataset bases (map-style and iterable): ``build()`` = load records + build the processor;
``get_collator()``; OpenAI-style record handling shared by every registered dataset.
Reference: src/lmms_engine/datasets/naive/base_dataset.py:11-122,
src/lmms_engine/datasets/iterable/base_iterable_dataset.py:11-110."""
from __future__ import annotations

import json
from typing import Any, Dict, List, Optional, Tuple

import torch

from ..mapping_func import DATAPROCESSOR_MAPPING
from ..utils.data_utils import DataUtilities
from ..utils.logging_utils import logger
from ..utils.train_utils import TrainUtilities
from .collator import PackedCollator, VisionCollator
from .config import DatasetConfig, ProcessorConfig
from .multimodal_mixin import MultiModalDataLoadingMixin


class DatasetCore(MultiModalDataLoadingMixin):
    """Loading of records, processor construction and per-record processing."""

    def __init__(self, config: DatasetConfig):
        self.config = config
        self.processor_config = (config.processor_config if isinstance(config.processor_config, ProcessorConfig)
                                 else ProcessorConfig(**(config.processor_config or {})))
        self.processor = None
        self.data_list: List[dict] = []
        self.data_folder: List[str] = []

    # ---- building -------------------------------------------------------------------------
    def build(self):
        self._build_from_config()
        self._build_processor()
        return self

    def _build_processor(self):
        name = self.processor_config.processor_type
        if name not in DATAPROCESSOR_MAPPING:
            raise KeyError(f"processor_type '{name}' is not registered; known: {sorted(DATAPROCESSOR_MAPPING)}")
        self.processor = DATAPROCESSOR_MAPPING[name](self.processor_config)
        self.processor.build()

    def _build_from_config(self):
        cfg = self.config
        fmt = cfg.dataset_format
        if cfg.datasets:
            self.data_list, self.data_folder = DataUtilities.load_inline_datasets(cfg.datasets)
        elif fmt == "yaml":
            self.data_list, self.data_folder = DataUtilities.load_yaml(cfg.dataset_path)
        elif fmt in ("json", "jsonl", "csv", "arrow", "parquet", "hf_dataset"):
            self.data_list = DataUtilities.load_one(cfg.dataset_path, fmt)
            self.data_folder = [""] * len(self.data_list)
        else:
            raise ValueError(f"unsupported dataset_format '{fmt}'")

    def load_from_json(self, path):
        return DataUtilities.load_json(path)

    def load_from_hf(self, path):
        return DataUtilities.load_one(path, "hf_dataset")

    # ---- one record -> model inputs ----------------------------------------------------------
    @staticmethod
    def messages_of(record: dict) -> List[dict]:
        msgs = record["messages"]
        if isinstance(msgs, str):  # parquet stores the list as a JSON string
            msgs = json.loads(msgs)
        return msgs

    def load_media(self, messages: List[dict], data_folder: Optional[str]) -> Tuple[list, list, list, list]:
        images, videos, audios, fps = [], [], [], []
        for m in messages:
            content = m["content"] if isinstance(m["content"], list) else []
            for c in content:
                t = c.get("type")
                if t == "image_url":
                    images.append(self.load_image(c["image_url"]["url"], data_folder))
                elif t == "video_url":
                    v = c["video_url"]
                    frames, f = self.load_video(v["url"], data_folder, v.get("video_start"), v.get("video_end"))
                    videos.append(frames)
                    fps.append(f)
                elif t == "audio_url":
                    audios.append(self.load_audio(c["audio_url"]["url"], data_folder=data_folder)[0])
        return images, videos, audios, fps

    def process_record(self, record: dict, data_folder: Optional[str] = "") -> Dict[str, torch.Tensor]:
        messages = self.messages_of(record)
        images, videos, audios, fps = self.load_media(messages, data_folder)
        hf_messages = TrainUtilities.convert_open_to_hf(messages)
        out = self.processor.process(hf_messages, images=images or None, videos=videos or None, audios=audios or None,
                                     video_fps=fps or None)
        if self.config.max_length and out["input_ids"].numel() > self.config.max_length:
            n = self.config.max_length
            for k in ("input_ids", "labels"):
                out[k] = out[k][:n]
            if "position_ids" in out:
                out["position_ids"] = out["position_ids"][..., :n]
        return out

    # ---- token-length estimate used by packing / filtering ---------------------------------------
    def estimate_tokens(self, record: dict) -> int:
        total = 0
        for m in self.messages_of(record):
            content = m["content"] if isinstance(m["content"], list) else [{"type": "text", "text": str(m["content"])}]
            for c in content:
                if c.get("precomputed_tokens") is not None:
                    total += int(c["precomputed_tokens"])
                elif c.get("type") == "image_url":
                    total += 2000
                elif c.get("type") == "audio_url":
                    total += 750
                elif c.get("type") == "video_url":
                    total += 5000
                elif c.get("type") == "text":
                    total += int(len(c.get("text", "").split()) * 1.5)
        return total

    def get_collator(self):
        kind = (self.config.extra_kwargs or {}).get("collator_type", "packed")
        if kind in ("vision", "padded"):
            return VisionCollator(self.processor)
        return PackedCollator()
