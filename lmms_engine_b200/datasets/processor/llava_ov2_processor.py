"""Processor of LLaVA-OneVision-2: every visual input becomes patch rows plus one ``(t, h, w)`` position per
patch (``patch_positions``), in the block layout the tower merges.

* images: resized to multiples of ``patch * merge``; positions are ``(0, row, column)``;
* plainly sampled videos (frames without codec metadata): every frame contributes all its patches at
  ``t = frame index``;
* codec-stream videos (``video_metadata`` holds objects with ``canvases`` / ``patch_positions`` /
  ``source_pts`` / ``fps``, see ``datasets/codec_video.py``): the canvases are cut into patches, unused cells
  are dropped, positions come from the codec, and the entry's grid is ``(kept blocks, merge, merge)``.

Videos are aliased into the image inputs (one entry of ``image_grid_thw`` per video, image placeholders in the
text), which is how the reference feeds its remote-code model
(src/lmms_engine/datasets/processor/llava_onevision2_processor.py:50-172, 264-343); each video's placeholders are
preceded by its duration and the number of sampled frames.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ...mapping_func import register_processor
from ...models.llava_ov2 import build_patch_positions
from ..codec_video import positions_to_block_layout
from . import vision_process as vp
from .chat import ChatProcessor


def looks_like_codec_output(obj) -> bool:
    return all(hasattr(obj, a) for a in ("canvases", "patch_positions", "source_pts", "fps"))


@register_processor("llava_onevision2")
class LlavaOnevision2Processor(ChatProcessor):
    temporal_patch_size = 1

    def build(self):
        super().build()
        self.patch_size = int(self.kwargs.get("patch_size", 14))
        self.merge_size = int(self.kwargs.get("merge_size", 2))
        return self

    # ---- patches ------------------------------------------------------------------------------------------
    def _frames_to_patches(self, frames: np.ndarray):
        """``frames [n, H, W, 3]`` (already sized) -> patch rows in block layout and the ``(n, gh, gw)`` grid."""
        return vp.patchify(frames, self.patch_size, 1, self.merge_size)

    def _image(self, img):
        arr = vp._to_array(img)
        h, w = vp.smart_resize(arr.shape[0], arr.shape[1], self.patch_size * self.merge_size,
                               self.kwargs.get("min_pixels", 56 * 56), self.kwargs.get("max_pixels", 14 * 14 * 4 * 1280))
        pix, grid = self._frames_to_patches(vp._resize(arr, h, w)[None])
        return pix, grid, build_patch_positions([grid], self.merge_size)

    def _plain_video(self, frames: np.ndarray):
        cfg = self.config
        h, w = vp.smart_resize(frames.shape[1], frames.shape[2], self.patch_size * self.merge_size,
                               getattr(cfg, "video_min_pixels", 3136) or 3136, getattr(cfg, "video_max_pixels", 768 * 28 * 28) or 768 * 28 * 28)
        frames = np.stack([vp._resize(f, h, w) for f in frames])
        pix, grid = self._frames_to_patches(frames)
        return pix, grid, build_patch_positions([grid], self.merge_size)

    def _codec_video(self, meta):
        canvases = np.asarray(meta.canvases)
        m, unit = self.merge_size, self.merge_size ** 2
        pix, grid = self._frames_to_patches(canvases)
        pos = positions_to_block_layout(np.asarray(meta.patch_positions), grid, m)
        if pos.shape[0] != pix.shape[0]:
            raise ValueError(f"codec patch_positions has {pos.shape[0]} rows, the canvases hold {pix.shape[0]} patches")
        used = pos[:, 0] >= 0
        if (used.reshape(-1, unit).all(1) != used.reshape(-1, unit).any(1)).any():
            raise ValueError("a merge block of a codec canvas is only partly used")
        keep = torch.from_numpy(np.nonzero(used)[0])
        n_blocks = int(used.sum()) // unit
        return pix.index_select(0, keep), (n_blocks, m, m), pos[used]

    # ---- text ---------------------------------------------------------------------------------------------
    def render_video(self, counters, mm) -> List[int]:
        i = counters["video"]
        counters["video"] += 1
        n = mm["video"][i]
        note = mm["video_notes"][i]
        return self._enc(note) + [self.vision_start] + [self.image_token_id] * n + [self.vision_end] + self._enc("\n")

    def process(self, hf_messages=None, images=None, videos=None, audios=None, add_system_prompt: bool = True,
                video_metadata: Optional[Sequence] = None, video_fps=None, **kw) -> Dict[str, torch.Tensor]:
        unit = self.merge_size ** 2
        entries = []  # (kind, pixels, grid, positions) in modality order: images first, then videos
        mm = {"image": [], "video": [], "audio": [], "video_notes": []}
        for img in images or []:
            pix, grid, pos = self._image(img)
            entries.append((pix, grid, pos))
            mm["image"].append(pix.shape[0] // unit)
        for i, vid in enumerate(videos or []):
            meta = video_metadata[i] if video_metadata and i < len(video_metadata) else None
            if meta is not None and looks_like_codec_output(meta):
                pix, grid, pos = self._codec_video(meta)
                pts = np.asarray(meta.source_pts, dtype=np.float64)
                note = f"<{float(pts.max() - pts.min()) if pts.size else 0.0:.1f} seconds, {pts.size} frames>"
            else:
                frames = np.asarray(vid)
                pix, grid, pos = self._plain_video(frames)
                fps = (video_fps[i] if video_fps and i < len(video_fps) else None) or float(getattr(self.config, "fps", 1) or 1)
                note = f"<{frames.shape[0] / fps:.1f} seconds, {frames.shape[0]} frames>"
            entries.append((pix, grid, pos))
            mm["video"].append(pix.shape[0] // unit)
            mm["video_notes"].append(note)
        out = self.build_ids_and_labels(hf_messages, mm, add_system_prompt)
        if entries:
            # the stream may interleave images and videos: placeholders are filled in order of appearance, so the
            # entries are ordered the way their runs appear in the text
            order = self._stream_order(hf_messages, len(images or []), len(videos or []))
            entries = [entries[j] for j in order]
            out["pixel_values"] = torch.cat([e[0] for e in entries], 0)
            out["image_grid_thw"] = torch.tensor([list(e[1]) for e in entries], dtype=torch.long)
            out["patch_positions"] = torch.from_numpy(np.concatenate([e[2] for e in entries], 0).astype(np.int64))
        return out

    @staticmethod
    def _stream_order(messages, n_images: int, n_videos: int) -> List[int]:
        order, ii, vi = [], 0, 0
        for m in messages or []:
            content = m["content"] if isinstance(m["content"], list) else []
            for c in content:
                if c.get("type") in ("image", "image_url") and ii < n_images:
                    order.append(ii)
                    ii += 1
                elif c.get("type") in ("video", "video_url") and vi < n_videos:
                    order.append(n_images + vi)
                    vi += 1
        return order
