"""Dataset section of the YAML (reference: src/lmms_engine/datasets/config.py:10-71)."""
from typing import List, Literal, Optional, Union

from pydantic import field_validator

from ..protocol import Args


class ProcessorConfig(Args):
    processor_name: str = ""
    processor_type: str = "pure_text"


class DatasetConfig(Args):
    dataset_type: str
    dataset_format: Literal["json", "jsonl", "csv", "yaml", "hf_dataset", "arrow", "parquet", "synthetic"] = "json"
    processor_config: Union[dict, ProcessorConfig] = {}
    dataset_path: Optional[str] = None
    datasets: Optional[List[dict]] = None
    shuffle: bool = True
    data_seed: Optional[int] = 42
    eval_dataset_path: Optional[str] = None
    object_storage: Optional[str] = "none"  # azure | gcs | none | a back end added with register_storage_backend
    bucket_name: Optional[str] = None
    packing: Optional[bool] = False
    packing_strategy: Optional[str] = None
    packing_length: Optional[int] = 32000
    filter_overlong: Optional[bool] = True
    filter_overlong_workers: Optional[int] = 8
    max_length: Optional[int] = None
    video_sampling_strategy: Optional[Literal["fps", "frame_num"]] = "fps"
    video_max_pixels: Optional[int] = 768 * 28 * 28
    video_max_frames: Optional[int] = 768
    video_min_pixels: Optional[int] = 3136
    frame_num: Optional[int] = 64
    fps: Optional[int] = 1
    video_backend: Optional[str] = "qwen_vl_utils"

    @field_validator(
        "video_max_pixels", "video_max_frames", "frame_num", "fps", "packing_length", "max_length",
        "filter_overlong_workers",
    )
    @classmethod
    def _positive(cls, v, info):
        if v is not None and v <= 0:
            raise ValueError(f"{info.field_name} must be positive, got {v}")
        return v

    @field_validator("video_backend")
    @classmethod
    def _backend(cls, v):
        if v == "torchvision":
            raise ValueError(
                "The 'torchvision' video backend has been removed; use 'decord', 'qwen_vl_utils' or 'qwen_omni_utils'."
            )
        if v not in (None, "decord", "qwen_vl_utils", "qwen_omni_utils", "lmms_video_utils"):
            raise ValueError(f"unknown video backend {v}")
        return v
