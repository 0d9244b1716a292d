"""Chat processors: OpenAI-style messages -> token ids, labels and multimodal tensors.

``ChatProcessor.process(hf_messages, images=None, videos=None, audios=None)`` renders every
message in ChatML (``<|im_start|>role\\n ... <|im_end|>\\n``), expands each image / video /
audio placeholder to the number of tokens its features occupy, and supervises assistant turns
only: user and system turns, the assistant header, and all multimodal placeholders are -100
(reference: ``get_qwen_template_labels``,
src/lmms_engine/datasets/processor/base_qwen2_5_processor.py:151-220; unlike the reference,
special tokens inside user turns stay masked).  Qwen3-VL style video rendering emits
``<t seconds>`` timestamps and one vision block per temporal step
(src/lmms_engine/datasets/processor/qwen3_vl_processor.py:179-220).
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Sequence

import numpy as np
import torch

from ...mapping_func import register_processor
from ...models import mrope
from . import vision_process as vp
from .tokenizer import load_tokenizer

IGNORE = -100


class ChatProcessor:
    """Text-only ChatML processor (``qwen2`` / ``pure_text`` and the base of the VL ones)."""

    patch_size, temporal_patch_size, merge_size = 14, 2, 2
    per_frame_video = False
    default_system = "You are a helpful assistant"

    def __init__(self, config):
        self.config = config
        self.kwargs = dict(getattr(config, "extra_kwargs", {}) or {})
        self.tokenizer = None

    def build(self):
        self.tokenizer = load_tokenizer(getattr(self.config, "processor_name", None))
        t = self.tokenizer
        self.im_start, self.im_end = t.convert_tokens_to_ids("<|im_start|>"), t.convert_tokens_to_ids("<|im_end|>")
        self.image_token_id = t.convert_tokens_to_ids("<|image_pad|>")
        self.video_token_id = t.convert_tokens_to_ids("<|video_pad|>")
        self.audio_token_id = t.convert_tokens_to_ids("<|AUDIO|>")
        self.vision_start = t.convert_tokens_to_ids("<|vision_start|>")
        self.vision_end = t.convert_tokens_to_ids("<|vision_end|>")
        return self

    @property
    def processor(self):
        return self

    def save_pretrained(self, path: str):
        self.tokenizer.save_pretrained(path)

    # ---- rendering ------------------------------------------------------------------------
    def _enc(self, text: str) -> List[int]:
        return list(self.tokenizer.encode(text, add_special_tokens=False))

    def render_message(self, msg: Dict[str, Any], counters: Dict[str, int], mm: Dict[str, List[int]]) -> List[int]:
        ids = self._enc(f"<|im_start|>{msg['role']}\n")
        content = msg["content"]
        if isinstance(content, str):
            content = [{"type": "text", "text": content}]
        for c in content:
            t = c.get("type")
            if t == "text":
                ids += self._enc(c["text"])
            elif t in ("image", "image_url"):
                n = mm["image"][counters["image"]]
                counters["image"] += 1
                ids += [self.vision_start] + [self.image_token_id] * n + [self.vision_end] + self._enc("\n")
            elif t in ("video", "video_url"):
                ids += self.render_video(counters, mm)
            elif t in ("audio", "audio_url"):
                n = mm["audio"][counters["audio"]]
                counters["audio"] += 1
                ids += [self.audio_token_id] * n + self._enc("\n")
        ids += [self.im_end] + self._enc("\n")
        return ids

    def render_video(self, counters, mm) -> List[int]:
        n = mm["video"][counters["video"]]
        counters["video"] += 1
        return [self.vision_start] + [self.video_token_id] * n + [self.vision_end] + self._enc("\n")

    def build_ids_and_labels(self, messages, mm, add_system_prompt=True) -> Dict[str, torch.Tensor]:
        counters = {"image": 0, "video": 0, "audio": 0, "frame": 0}
        ids: List[int] = []
        labels: List[int] = []
        if add_system_prompt and messages and messages[0]["role"] != "system":
            sys_ids = self.render_message({"role": "system", "content": self.default_system}, counters, mm)
            ids += sys_ids
            labels += [IGNORE] * len(sys_ids)
        header = len(self._enc("<|im_start|>assistant\n"))
        for msg in messages:
            enc = self.render_message(msg, counters, mm)
            ids += enc
            if msg["role"] == "assistant":
                labels += [IGNORE] * header + enc[header:]
            else:
                labels += [IGNORE] * len(enc)
        ids_t = torch.tensor(ids, dtype=torch.long)
        lab_t = torch.tensor(labels, dtype=torch.long)
        for tok in (self.image_token_id, self.video_token_id, self.audio_token_id):
            if tok is not None:
                lab_t[ids_t == tok] = IGNORE
        return {"input_ids": ids_t, "labels": lab_t}

    def process(self, hf_messages=None, images=None, videos=None, audios=None, add_system_prompt: bool = True, **kw):
        return self.build_ids_and_labels(hf_messages, {"image": [], "video": [], "audio": []}, add_system_prompt)


for _name in ("qwen2", "pure_text", "qwen3"):
    register_processor(_name)(ChatProcessor)


class QwenVLProcessor(ChatProcessor):
    """Qwen2-VL / Qwen2.5-VL: images and videos become patch rows; every 2x2 block of patches
    is one placeholder token; multimodal rotary positions are attached."""

    tokens_per_second = 2.0

    def process(self, hf_messages=None, images=None, videos=None, audios=None, add_system_prompt: bool = True,
                video_fps: Optional[Sequence[float]] = None, **kw):
        cfg = self.config
        out: Dict[str, torch.Tensor] = {}
        mm = {"image": [], "video": [], "audio": [], "video_grids": []}
        unit = self.merge_size ** 2
        grids, secs = [], []
        kw_img = dict(patch=self.patch_size, temporal=self.temporal_patch_size, merge=self.merge_size)
        if images:
            pix, g = vp.process_images(images, min_pixels=self.kwargs.get("min_pixels", 56 * 56),
                                       max_pixels=self.kwargs.get("max_pixels", 14 * 14 * 4 * 1280), **kw_img)
            out["pixel_values"], out["image_grid_thw"] = pix, g
            mm["image"] = [int(t * h * w) // unit for t, h, w in g.tolist()]
        if videos:
            pv, gv, spg = [], [], []
            for i, frames in enumerate(videos):
                p, g = vp.process_video(np.asarray(frames), min_pixels=getattr(cfg, "video_min_pixels", 3136) or 3136,
                                        max_pixels=getattr(cfg, "video_max_pixels", 768 * 28 * 28) or 768 * 28 * 28, **kw_img)
                pv.append(p)
                gv.append(g)
                fps = (video_fps[i] if video_fps else None) or float(getattr(cfg, "fps", 1) or 1)
                spg.append(self.temporal_patch_size / fps)
            out["pixel_values_videos"], out["video_grid_thw"] = torch.cat(pv), torch.cat(gv)
            out["second_per_grid_ts"] = torch.tensor(spg, dtype=torch.float32)
            mm["video_grids"] = out["video_grid_thw"].tolist()
            mm["video"] = [int(t * h * w) // unit for t, h, w in mm["video_grids"]]
        out.update(self.build_ids_and_labels(hf_messages, mm, add_system_prompt))
        out["position_ids"] = self.positions(out)
        return out

    def positions(self, out) -> torch.Tensor:
        ids = out["input_ids"]
        grids, secs = self._grids_in_stream_order(out)
        cu = [0, ids.numel()]
        return mrope.build_mrope_positions(ids, cu, (self.image_token_id, self.video_token_id), grids, secs,
                                           self.merge_size, self.tokens_per_second)

    def _grids_in_stream_order(self, out):
        ids = out["input_ids"].tolist()
        img = out["image_grid_thw"].tolist() if "image_grid_thw" in out else []
        vid = out["video_grid_thw"].tolist() if "video_grid_thw" in out else []
        spg = out["second_per_grid_ts"].tolist() if "second_per_grid_ts" in out else []
        grids, secs, ii, vi, prev = [], [], 0, 0, None
        for t in ids:
            if t == self.image_token_id and prev != t:
                grids.append(img[ii]); secs.append(0.0); ii += 1
            elif t == self.video_token_id and prev != t:
                g = vid[vi]
                if self.per_frame_video:
                    grids.append([1, g[1], g[2]]); secs.append(0.0)
                    self._frame_left = getattr(self, "_frame_left", g[0]) - 1
                    if self._frame_left == 0:
                        vi += 1
                        del self._frame_left
                else:
                    grids.append(g); secs.append(spg[vi]); vi += 1
            prev = t
        return grids, secs


for _name in ("qwen2_vl", "qwen2_5_vl"):
    register_processor(_name)(QwenVLProcessor)


@register_processor("qwen3_vl")
class Qwen3VLProcessor(QwenVLProcessor):
    """Qwen3-VL: 16-pixel patches; a video is written frame group by frame group as
    ``<t seconds><|vision_start|>...<|vision_end|>`` so every group has temporal extent 1."""

    patch_size = 16
    per_frame_video = True
    tokens_per_second = 0.0

    def process(self, hf_messages=None, images=None, videos=None, audios=None, add_system_prompt: bool = True,
                video_fps=None, video_metadata=None, **kw):
        """``video_metadata``: one dict per video with ``frame_times`` (seconds of every sampled frame, what the
        Qwen3-VL dataset reads from the decoder) or ``fps`` + ``frames_indices``; without it the timestamps assume
        frames sampled at the configured (or ``video_fps``) rate."""
        self._video_times = []
        for i in range(len(videos or [])):
            meta = (video_metadata[i] if video_metadata and i < len(video_metadata) else None) or {}
            if meta.get("frame_times") is not None:
                self._video_times.append([float(x) for x in meta["frame_times"]])
            elif meta.get("frames_indices") is not None and meta.get("fps"):
                self._video_times.append([float(ix) / float(meta["fps"]) for ix in meta["frames_indices"]])
            else:
                self._video_times.append(None)
        self._video_fps = list(video_fps) if video_fps else []
        try:
            return super().process(hf_messages, images=images, videos=videos, audios=audios, add_system_prompt=add_system_prompt,
                                   video_fps=video_fps, **kw)
        finally:
            self._video_times, self._video_fps = [], []

    def render_video(self, counters, mm) -> List[int]:
        i = counters["video"]
        counters["video"] += 1
        t, h, w = mm["video_grids"][i]
        per = (h * w) // (self.merge_size ** 2)
        times = getattr(self, "_video_times", None)
        times = times[i] if times and i < len(times) else None
        fps_list = getattr(self, "_video_fps", None) or []
        fps = float((fps_list[i] if i < len(fps_list) else None) or getattr(self.config, "fps", 1) or 1)
        ids: List[int] = []
        for f in range(t):
            if times:
                # mean time of the frames merged into this temporal step (the last frame repeats when the count is odd)
                group = [times[min(f * self.temporal_patch_size + j, len(times) - 1)] for j in range(self.temporal_patch_size)]
                stamp = sum(group) / len(group)
            else:
                stamp = (f * self.temporal_patch_size + (self.temporal_patch_size - 1) / 2.0) / fps
            ids += self._enc(f"<{stamp:.1f} seconds>")
            ids += [self.vision_start] + [self.video_token_id] * per + [self.vision_end]
        return ids + self._enc("\n")
