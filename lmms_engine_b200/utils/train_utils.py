"""Small training helpers: device tables, formatters, pytree device moves
(reference: src/lmms_engine/utils/train_utils.py:21-520; ``send_to_device`` comes from
accelerate there)."""
from __future__ import annotations

from typing import Any, Dict, Mapping

import torch

_PEAK_FLOPS = [
    ("B200", 2.25e15), ("B300", 2.25e15), ("GB200", 2.25e15), ("MI300X", 1336e12), ("H100", 989e12), ("H800", 989e12),
    ("H200", 989e12), ("A100", 312e12), ("A800", 312e12), ("L40", 181.05e12), ("L20", 119.5e12), ("H20", 148e12),
    ("910B", 354e12), ("A6000", 154.8e12), ("RTX 3070 Ti", 21.75e12),
]
_TDP = [("MI300X", 750.0), ("B200", 1000.0), ("B300", 1200.0), ("H100", 700.0), ("H800", 700.0), ("H200", 700.0),
        ("A100", 400.0), ("A800", 400.0), ("L40", 300.0), ("H20", 400.0), ("A6000", 300.0)]


class TrainUtilities:
    @staticmethod
    def _device_name() -> str:
        return torch.cuda.get_device_name() if torch.cuda.is_available() else "cpu"

    @staticmethod
    def get_device_flops(unit: str = "T") -> float:
        name = TrainUtilities._device_name()
        flops = float("inf")
        for key, val in _PEAK_FLOPS:
            if key in name:
                flops = val
                break
        div = {"B": 1.0, "K": 1e3, "M": 1e6, "G": 1e9, "T": 1e12, "P": 1e15}[unit]
        return flops / div

    @staticmethod
    def get_device_tdp() -> float:
        name = TrainUtilities._device_name()
        for key, val in _TDP:
            if key in name:
                return val
        return 0.0

    @staticmethod
    def format_tokens(n: float) -> str:
        for unit, div in (("T", 1e12), ("B", 1e9), ("M", 1e6), ("K", 1e3)):
            if abs(n) >= div:
                return f"{n / div:.2f}{unit}"
        return f"{n:.0f}"

    @staticmethod
    def format_flops(n: float) -> str:
        for unit, div in (("ZFLOPs", 1e21), ("EFLOPs", 1e18), ("PFLOPs", 1e15), ("TFLOPs", 1e12), ("GFLOPs", 1e9)):
            if abs(n) >= div:
                return f"{n / div:.2f} {unit}"
        return f"{n:.0f} FLOPs"

    @staticmethod
    def convert_open_to_hf(messages):
        """OpenAI-style content parts -> HF chat-template parts (image_url -> image ...)."""
        out = []
        for m in messages:
            parts = []
            for c in m["content"]:
                t = c["type"]
                if t == "text":
                    parts.append({"type": "text", "text": c["text"]})
                elif t == "image_url":
                    parts.append({"type": "image", "image": c["image_url"]["url"]})
                elif t == "audio_url":
                    parts.append({"type": "audio", "audio": c["audio_url"]["url"]})
                elif t == "video_url":
                    parts.append({"type": "video", "video": c["video_url"]["url"]})
                else:
                    parts.append(c)
            out.append({"role": m["role"], "content": parts})
        return out


def send_to_device(obj: Any, device, non_blocking: bool = True) -> Any:
    if torch.is_tensor(obj):
        return obj.to(device, non_blocking=non_blocking)
    if isinstance(obj, Mapping):
        return type(obj)({k: send_to_device(v, device, non_blocking) for k, v in obj.items()})
    if isinstance(obj, (list, tuple)):
        return type(obj)(send_to_device(v, device, non_blocking) for v in obj)
    return obj


def str_to_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        return name
    return {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float16": torch.float16, "fp16": torch.float16,
            "float32": torch.float32, "fp32": torch.float32}[str(name).replace("torch.", "")]
