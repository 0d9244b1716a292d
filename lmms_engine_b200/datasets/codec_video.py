"""Codec-stream videos for LLaVA-OneVision-2: instead of sampling whole frames, keep every patch block
of the key frames and, of the frames in between, only the blocks that changed - the way a video codec
spends bits - and pack the kept blocks into fixed-size canvases.  Every kept patch carries its
``(t, h, w)`` position in the source video, which the vision tower uses for its rotary embedding, so
the canvases are only a transport format.

The reference obtains the same triple (canvases, patch positions, frame times) from the external
``lmms_video_utils`` codec back end and feeds it to the OV2 processor
(src/lmms_engine/datasets/codec_video_mixin.py:17-71,
src/lmms_engine/datasets/processor/llava_onevision2_processor.py:228-343,
src/lmms_engine/datasets/iterable/llava_ov2_iterable_dataset.py:17-56).  Here the selection is part of
the engine (``select_codec_patches``), a back end with the ``lmms_video_utils`` interface is used when it
is installed, and the dataset mixin / dataset class below have the reference's names and roles.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

import numpy as np

from ..mapping_func import register_dataset
from .iterable.multimodal_iterable_dataset import MultiModalIterableDataset


@dataclass
class CodecVideoOutput:
    """``canvases [n, H, W, 3] uint8`` hold the kept blocks in raster order (unused cells are zero);
    ``patch_positions [n * (H/p) * (W/p), 3]`` gives ``(t, h, w)`` of every canvas patch in raster order of the
    canvases (``-1`` rows mark unused cells); ``source_pts`` are the times of the sampled frames in seconds."""

    canvases: np.ndarray
    patch_positions: np.ndarray
    source_pts: np.ndarray
    fps: float
    grid_hw: Tuple[int, int] = (0, 0)  # patch grid of a source frame
    kept_blocks: int = 0
    total_blocks: int = 0


def select_codec_patches(frames: np.ndarray, patch: int = 14, merge: int = 2, keyframe_interval: int = 8,
                         threshold: float = 6.0, canvas_blocks: Tuple[int, int] = (16, 16), times: Optional[np.ndarray] = None,
                         fps: float = 1.0, max_blocks: Optional[int] = None) -> CodecVideoOutput:
    """``frames [n, H, W, 3] uint8`` with H, W multiples of ``patch * merge``.

    A block is ``merge x merge`` patches.  Frame 0 and every ``keyframe_interval``-th frame keep all blocks; another
    frame keeps a block when its mean absolute difference to the LAST KEPT version of that block exceeds
    ``threshold`` (grey levels).  ``max_blocks`` keeps the largest residuals of the non-key frames when the budget is
    exceeded."""
    n, H, W, _ = frames.shape
    b = patch * merge
    if H % b or W % b:
        raise ValueError(f"frame size {(H, W)} must be a multiple of patch * merge = {b}")
    gh, gw = H // b, W // b
    blocks = frames.reshape(n, gh, b, gw, b, 3).transpose(0, 1, 3, 2, 4, 5).astype(np.float32)  # n, gh, gw, b, b, 3
    ref = blocks[0].copy()
    keep: List[Tuple[int, int, int, float]] = []
    for t in range(n):
        if t % max(keyframe_interval, 1) == 0:
            keep += [(t, i, j, np.inf) for i in range(gh) for j in range(gw)]
            ref = blocks[t].copy()
            continue
        resid = np.abs(blocks[t] - ref).mean(axis=(2, 3, 4))
        for i, j in zip(*np.nonzero(resid > threshold)):
            keep.append((t, int(i), int(j), float(resid[i, j])))
            ref[i, j] = blocks[t, i, j]
    if max_blocks is not None and len(keep) > max_blocks:
        keyed = [k for k in keep if k[3] == np.inf]
        rest = sorted((k for k in keep if k[3] != np.inf), key=lambda k: -k[3])[: max(max_blocks - len(keyed), 0)]
        keep = sorted(keyed + rest, key=lambda k: (k[0], k[1], k[2]))
    ch, cw = canvas_blocks
    per = ch * cw
    n_canvas = max(-(-len(keep) // per), 1)
    canvases = np.zeros((n_canvas, ch * b, cw * b, 3), dtype=np.uint8)
    pos = np.full((n_canvas, ch * merge, cw * merge, 3), -1, dtype=np.int64)
    for idx, (t, i, j, _) in enumerate(keep):
        c, r = divmod(idx, per)
        bi, bj = divmod(r, cw)
        canvases[c, bi * b:(bi + 1) * b, bj * b:(bj + 1) * b] = frames[t, i * b:(i + 1) * b, j * b:(j + 1) * b]
        for di in range(merge):
            for dj in range(merge):
                pos[c, bi * merge + di, bj * merge + dj] = (t, i * merge + di, j * merge + dj)
    pts = np.asarray(times, dtype=np.float64) if times is not None else np.arange(n, dtype=np.float64) / max(fps, 1e-6)
    return CodecVideoOutput(canvases=canvases, patch_positions=pos.reshape(-1, 3), source_pts=pts, fps=float(fps),
                            grid_hw=(gh * merge, gw * merge), kept_blocks=len(keep), total_blocks=n * gh * gw)


def positions_to_block_layout(pos: np.ndarray, grid: Tuple[int, int, int], merge: int) -> np.ndarray:
    """Reorder per-patch rows from raster order of ``(t, h, w)`` canvases to the tower's order, in which the
    ``merge x merge`` patches of a block are adjacent."""
    t, h, w = grid
    x = pos.reshape(t, h // merge, merge, w // merge, merge, -1).transpose(0, 1, 3, 2, 4, 5)
    return x.reshape(t * h * w, -1)


class CodecVideoLoadingMixin:
    """Collects codec-stream video inputs from OpenAI-style messages (expects ``load_video_with_metadata`` and a
    ``config`` from the host class)."""

    def load_codec_video(self, video_path: str, data_folder: Optional[str] = None, video_kwargs: Optional[Dict[str, Any]] = None):
        kw = dict((self.config.extra_kwargs or {}).get("codec", {}) or {})
        kw.update(video_kwargs or {})
        try:  # an installed back end with the reference's interface takes precedence
            import lmms_video_utils  # type: ignore

            full = self._resolve(video_path, data_folder)
            out = lmms_video_utils.load_video(full, fps=self.config.fps, **kw)
            return out.canvases, float(out.fps), out
        except ImportError:
            pass
        frames, meta = self.load_video_with_metadata(video_path, data_folder, kw.pop("video_start", None), kw.pop("video_end", None))
        patch, merge = int(kw.pop("patch_size", 14)), int(kw.pop("merge_size", 2))
        b = patch * merge
        size = kw.pop("frame_size", None)
        H = W = None
        if size:
            H, W = (int(size), int(size)) if np.isscalar(size) else (int(size[0]), int(size[1]))
        else:
            H, W = max(frames.shape[1] // b, 1) * b, max(frames.shape[2] // b, 1) * b
        if (H, W) != frames.shape[1:3]:
            from PIL import Image

            frames = np.stack([np.asarray(Image.fromarray(f).resize((W, H), Image.BICUBIC)) for f in frames])
        out = select_codec_patches(frames, patch=patch, merge=merge, times=np.asarray(meta["frame_times"]), fps=meta["sample_fps"], **kw)
        return out.canvases, float(meta["sample_fps"]), out

    def collect_codec_video_inputs(self, messages: List[dict], data_folder: Optional[str] = None):
        """``(videos, metadata, fps)``: canvases and their ``CodecVideoOutput`` for every ``video_url`` of the messages."""
        videos, metas, fps = [], [], None
        for m in messages:
            for c in (m["content"] if isinstance(m["content"], list) else []):
                if c.get("type") != "video_url":
                    continue
                v = c["video_url"]
                extra = {k: val for k, val in v.items() if k != "url" and val is not None}
                canvases, fps, out = self.load_codec_video(v["url"], data_folder, extra or None)
                videos.append(canvases)
                metas.append(out)
        return videos, metas, fps


@register_dataset("llava_ov2_iterable")
class LlavaOV2IterableDataset(CodecVideoLoadingMixin, MultiModalIterableDataset):
    """Streaming dataset of LLaVA-OneVision-2: images as usual, videos as codec streams."""

    def process_record(self, record: dict, data_folder: Optional[str] = ""):
        from ..utils.train_utils import TrainUtilities

        messages = self.messages_of(record)
        images = [self.load_image(c["image_url"]["url"], data_folder) for m in messages
                  for c in (m["content"] if isinstance(m["content"], list) else []) if c.get("type") == "image_url"]
        videos, metas, fps = self.collect_codec_video_inputs(messages, data_folder)
        hf_messages = TrainUtilities.convert_open_to_hf(messages)
        out = self.processor.process(hf_messages, images=images or None, videos=videos or None, video_metadata=metas or None,
                                     video_fps=[fps] * len(videos) if videos else None)
        if self.config.max_length and out["input_ids"].numel() > self.config.max_length:
            raise ValueError("a LLaVA-OneVision-2 sample cannot be truncated (placeholders and patches must stay aligned); "
                             f"raise max_length above {out['input_ids'].numel()} or lower the codec budget")
        return out
