"""Image / video preprocessing for the Qwen-VL families without external image processors:
``smart_resize`` (both sides multiples of ``patch*merge``, area within ``[min_pixels,
max_pixels]``, aspect ratio kept), normalisation, and flattening into patch rows in the order
``(grid_t, grid_h/m, grid_w/m, m, m, C, T_p, p, p)`` -> ``pixel_values [P, C*T_p*p*p]``.
Upstream behaviour: ``transformers`` ``Qwen2VLImageProcessor`` / video processors (see the
patch-order note in the reference processors, src/lmms_engine/datasets/processor/base_qwen2_5_processor.py:139-149)."""
from __future__ import annotations

import math
from typing import List, Sequence, Tuple

import numpy as np
import torch

CLIP_MEAN = (0.48145466, 0.4578275, 0.40821073)
CLIP_STD = (0.26862954, 0.26130258, 0.27577711)


def smart_resize(height: int, width: int, factor: int = 28, min_pixels: int = 56 * 56, max_pixels: int = 14 * 14 * 4 * 1280) -> Tuple[int, int]:
    if max(height, width) / max(min(height, width), 1) > 200:
        raise ValueError("absolute aspect ratio must be smaller than 200")
    h = max(factor, round(height / factor) * factor)
    w = max(factor, round(width / factor) * factor)
    if h * w > max_pixels:
        beta = math.sqrt((height * width) / max_pixels)
        h = max(factor, math.floor(height / beta / factor) * factor)
        w = max(factor, math.floor(width / beta / factor) * factor)
    elif h * w < min_pixels:
        beta = math.sqrt(min_pixels / (height * width))
        h = math.ceil(height * beta / factor) * factor
        w = math.ceil(width * beta / factor) * factor
    return h, w


def _to_array(img) -> np.ndarray:
    if isinstance(img, np.ndarray):
        return img
    if torch.is_tensor(img):
        return img.numpy()
    return np.asarray(img.convert("RGB"))


def _resize(arr: np.ndarray, h: int, w: int) -> np.ndarray:
    if arr.shape[0] == h and arr.shape[1] == w:
        return arr
    from PIL import Image

    return np.asarray(Image.fromarray(arr).resize((w, h), Image.BICUBIC))


def patchify(frames: np.ndarray, patch: int, temporal: int, merge: int, mean=CLIP_MEAN, std=CLIP_STD):
    """``frames [n, H, W, 3] uint8`` (H, W multiples of patch*merge) -> (pixel_values, (t, h, w))."""
    n = frames.shape[0]
    if n % temporal:
        frames = np.concatenate([frames, np.repeat(frames[-1:], temporal - n % temporal, 0)], 0)
    x = frames.astype(np.float32) / 255.0
    x = (x - np.asarray(mean, np.float32)) / np.asarray(std, np.float32)
    x = x.transpose(0, 3, 1, 2)  # [n, C, H, W]
    n, C, H, W = x.shape
    gt, gh, gw = n // temporal, H // patch, W // patch
    x = x.reshape(gt, temporal, C, gh // merge, merge, patch, gw // merge, merge, patch)
    x = x.transpose(0, 3, 6, 4, 7, 2, 1, 5, 8)  # gt, gh/m, gw/m, m, m, C, Tp, p, p
    return torch.from_numpy(np.ascontiguousarray(x.reshape(gt * gh * gw, C * temporal * patch * patch))), (gt, gh, gw)


def process_images(images: Sequence, patch: int = 14, temporal: int = 2, merge: int = 2, min_pixels: int = 56 * 56,
                   max_pixels: int = 14 * 14 * 4 * 1280):
    pix, grids = [], []
    for img in images:
        arr = _to_array(img)
        h, w = smart_resize(arr.shape[0], arr.shape[1], patch * merge, min_pixels, max_pixels)
        arr = _resize(arr, h, w)
        p, g = patchify(np.repeat(arr[None], temporal, 0), patch, temporal, merge)
        pix.append(p)
        grids.append(g)
    return torch.cat(pix, 0), torch.tensor(grids, dtype=torch.long)


def process_video(frames: np.ndarray, patch: int = 14, temporal: int = 2, merge: int = 2, min_pixels: int = 3136,
                  max_pixels: int = 768 * 28 * 28):
    h, w = smart_resize(frames.shape[1], frames.shape[2], patch * merge, min_pixels, max_pixels)
    frames = np.stack([_resize(f, h, w) for f in frames])
    p, g = patchify(frames, patch, temporal, merge)
    return p, torch.tensor([g], dtype=torch.long)
