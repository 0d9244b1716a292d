"""Processors of the generative families, one per family because their pixel contracts differ:

* ``sit``: ADM centre crop (box-halve while the short side is at least twice the target, bicubic to the target short
  side, crop the centre), random horizontal flip, pixels in ``[-1, 1]``, class label passed through
  (src/lmms_engine/datasets/processor/sit_processor.py:10-55);
* ``rae_siglip``: resize to a square 1.5 x the encoder size (384 for 256), random crop of the encoder size, pixels in
  ``[0, 1]`` - the autoencoder applies its encoder's statistics itself; one placeholder id per latent token
  (src/lmms_engine/datasets/processor/rae_processor.py:15-86);
* ``wanvideo``: the caption of the first message tokenised (at most 256 tokens), frames resized with a Lanczos filter,
  centre-cropped and scaled to ``[-1, 1]``, returned as ``video [T, H, W, C]`` like the reference
  (src/lmms_engine/datasets/processor/wanvideo_processor.py:11-86,
  src/lmms_engine/models/wanvideo/processing_wanvideo.py:17-212); the padded collator stacks clips into ``[B, T, H, W, C]``.
"""
from __future__ import annotations

import os
import random
from typing import Any, Dict, List, Optional, Sequence

import numpy as np
import torch

from ...mapping_func import register_processor
from .tokenizer import load_tokenizer


class _PixelProcessor:
    def __init__(self, config):
        self.config = config
        self.kwargs = dict(getattr(config, "extra_kwargs", {}) or {})
        self.tokenizer = None

    def build(self):
        return self

    @property
    def processor(self):
        return self

    def save_pretrained(self, path: str):
        os.makedirs(path, exist_ok=True)
        if self.tokenizer is not None and hasattr(self.tokenizer, "save_pretrained"):
            self.tokenizer.save_pretrained(path)

    @staticmethod
    def to_pil(img):
        from PIL import Image

        if not isinstance(img, Image.Image):
            img = Image.fromarray(np.asarray(img).astype(np.uint8))
        return img.convert("RGB")

    @staticmethod
    def to_unit_tensor(img) -> torch.Tensor:
        return torch.from_numpy(np.asarray(img).copy()).permute(2, 0, 1).float() / 255.0


def adm_center_crop(img, size: int):
    from PIL import Image

    while min(img.size) >= 2 * size:
        img = img.resize(tuple(x // 2 for x in img.size), resample=Image.BOX)
    scale = size / min(img.size)
    img = img.resize(tuple(round(x * scale) for x in img.size), resample=Image.BICUBIC)
    w, h = img.size
    left, top = (w - size) // 2, (h - size) // 2
    return img.crop((left, top, left + size, top + size))


@register_processor("sit")
class SitProcessor(_PixelProcessor):
    def build(self):
        self.image_size = int(self.kwargs.get("image_size", 256))
        self.flip = bool(self.kwargs.get("random_flip", True))
        return self

    def image_to_tensor(self, img) -> torch.Tensor:
        x = self.to_unit_tensor(adm_center_crop(self.to_pil(img), self.image_size))
        if self.flip and random.random() < 0.5:
            x = x.flip(-1)
        return (x - 0.5) / 0.5

    def process(self, image=None, label: Optional[int] = None, **kw):
        out = {"pixel_values": self.image_to_tensor(image)}
        if label is not None:
            out["labels"] = torch.tensor(int(label))
        return out


@register_processor("rae_siglip")
class RaeSiglipProcessor(_PixelProcessor):
    def build(self):
        self.image_size = int(self.kwargs.get("image_size", 256))
        self.patch_size = int(self.kwargs.get("patch_size", 16))
        self.num_tokens = (self.image_size // self.patch_size) ** 2
        self.first_crop_size = int(self.kwargs.get("first_crop_size", 384 if self.image_size == 256 else round(self.image_size * 1.5)))
        return self

    def image_to_tensor(self, img) -> torch.Tensor:
        from PIL import Image

        s, c = self.first_crop_size, self.image_size
        img = self.to_pil(img).resize((s, s), resample=Image.BICUBIC)
        left, top = (random.randint(0, s - c), random.randint(0, s - c)) if s > c else (0, 0)
        return self.to_unit_tensor(img.crop((left, top, left + c, top + c)))

    def process(self, image=None, images: Optional[Sequence] = None, **kw):
        if images is not None:
            px = torch.stack([self.image_to_tensor(i) for i in images])
            ids = torch.ones(px.shape[0], self.num_tokens, dtype=torch.long)
            return {"pixel_values": px, "input_ids": ids, "attention_mask": torch.ones_like(ids)}
        return {"pixel_values": self.image_to_tensor(image)}


@register_processor("wanvideo")
class WanVideoProcessor(_PixelProcessor):
    max_text_len = 256

    def build(self):
        kw = self.kwargs
        size = kw.get("size") or {"height": 480, "width": 832}
        crop = kw.get("crop_size") or size
        self.size, self.crop = (int(size["height"]), int(size["width"])), (int(crop["height"]), int(crop["width"]))
        self.do_resize, self.do_center_crop = bool(kw.get("do_resize", True)), bool(kw.get("do_center_crop", True))
        self.mean = np.asarray(kw.get("image_mean") or [0.5, 0.5, 0.5], dtype=np.float32).reshape(1, 1, 3)
        self.std = np.asarray(kw.get("image_std") or [0.5, 0.5, 0.5], dtype=np.float32).reshape(1, 1, 3)
        self.tokenizer = load_tokenizer(getattr(self.config, "processor_name", None))
        return self

    def frame(self, img) -> np.ndarray:
        from PIL import Image

        img = self.to_pil(img)
        if self.do_resize:
            img = img.resize((self.size[1], self.size[0]), Image.LANCZOS)
        arr = np.asarray(img)
        if self.do_center_crop:
            h, w = arr.shape[:2]
            top, left = (h - self.crop[0]) // 2, (w - self.crop[1]) // 2
            arr = arr[top:top + self.crop[0], left:left + self.crop[1]]
        return (arr.astype(np.float32) / 255.0 - self.mean) / self.std

    @staticmethod
    def prompt_of(hf_messages) -> str:
        """The caption: the first text part of the first message (no chat template)."""
        if not hf_messages:
            return ""
        if isinstance(hf_messages, str):
            return hf_messages
        content = hf_messages[0]["content"]
        if isinstance(content, str):
            return content
        return next((c["text"] for c in content if c.get("type") == "text"), "")

    def process(self, hf_messages=None, images=None, videos=None, **kw) -> Dict[str, Any]:
        if not videos:
            raise ValueError("a video sample needs frames")
        frames = videos[0] if isinstance(videos[0], (list, tuple)) or (hasattr(videos[0], "ndim") and videos[0].ndim == 4) else videos
        keep = 1 + (len(frames) - 1) // 4 * 4  # the autoencoder takes 1 + 4k frames
        video = torch.from_numpy(np.stack([self.frame(f) for f in list(frames)[:keep]]))  # T, H, W, C
        ids = list(self.tokenizer.encode(self.prompt_of(hf_messages), add_special_tokens=False))[: self.max_text_len]
        ids_t = torch.tensor(ids or [0], dtype=torch.long)
        return {"video": video, "input_ids": ids_t}
