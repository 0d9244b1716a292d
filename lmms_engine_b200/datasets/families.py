"""Dataset classes whose record handling differs from the generic multimodal datasets.

Each behaviour is a mixin over ``DatasetCore`` and is registered twice, as a map-style and as a
streaming dataset, under the names the reference uses:

* ``qwen3_vl`` / ``qwen3_vl_iterable`` - videos are decoded TOGETHER with their metadata (source fps, the
  indices of the sampled frames), which the Qwen3-VL processor turns into the ``<t seconds>`` stamps it
  writes before every temporal step; frames are never re-sampled by the processor
  (reference: src/lmms_engine/datasets/naive/qwen3_vl_dataset.py:16-122,
  iterable/qwen3_vl_iterable_dataset.py).
* ``qwen_omni`` / ``qwen_omni_iterable`` - audio clips longer than the processor's ``audio_max_length``
  seconds are split into that many placeholders; a video may contribute its own sound track
  (``use_audio_in_video``), whose chunks are interleaved with the video tokens
  (reference: src/lmms_engine/datasets/iterable/qwen_omni_iterable_dataset.py:20-152,
  naive/qwen_omni_dataset.py).
* ``llava_video`` - time-aware video loading for LLaVA-Video: an upper bound on the frame count with
  optional forced uniform sampling, frame directories as videos, CSV rows ``video,prompt[,answer]``, an optional
  time instruction ("The video lasts for ... seconds ...") put in front of the first user turn, and the
  slow-fast pooling options handed to the processor
  (reference: src/lmms_engine/datasets/naive/llava_video_dataset.py:17-494).
* ``vision`` / ``vision_audio`` / ``text`` (and their iterable forms) keep the generic record handling.
"""
from __future__ import annotations

import copy
import os
from typing import Any, Dict, List, Optional, Tuple

import numpy as np
import torch

from ..mapping_func import register_dataset
from ..utils.logging_utils import logger
from ..utils.train_utils import TrainUtilities
from .iterable.multimodal_iterable_dataset import MultiModalIterableDataset
from .naive.multimodal_dataset import MultiModalDataset

IMAGE_SUFFIXES = (".jpg", ".jpeg", ".png", ".bmp", ".webp")


def _truncate(cfg, out: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    if cfg.max_length and out["input_ids"].numel() > cfg.max_length:
        n = cfg.max_length
        for k in ("input_ids", "labels"):
            out[k] = out[k][:n]
        if "position_ids" in out:
            out["position_ids"] = out["position_ids"][..., :n]
    return out


# ------------------------------------------------------------------------------------------------ Qwen3-VL
class Qwen3VLRecords:
    """Video frames travel with the times at which they were taken."""

    def process_record(self, record: dict, data_folder: Optional[str] = "") -> Dict[str, torch.Tensor]:
        messages = self.messages_of(record)
        images, videos, metas, fps = [], [], [], []
        for m in messages:
            for c in (m["content"] if isinstance(m["content"], list) else []):
                if c.get("type") == "image_url":
                    images.append(self.load_image(c["image_url"]["url"], data_folder))
                elif c.get("type") == "video_url":
                    v = c["video_url"]
                    frames, meta = self.load_video_with_metadata(v["url"], data_folder, v.get("video_start"), v.get("video_end"))
                    videos.append(frames)
                    metas.append(meta)
                    fps.append(meta["sample_fps"])
        hf_messages = TrainUtilities.convert_open_to_hf(messages)
        out = self.processor.process(hf_messages, images=images or None, videos=videos or None, video_fps=fps or None,
                                     video_metadata=metas or None, do_sample_frames=False)
        return _truncate(self.config, out)


# ------------------------------------------------------------------------------------------------ Qwen-Omni
class QwenOmniRecords:
    """Audio chunking and sound tracks of videos."""

    DEFAULT_MAX_AUDIO_SECONDS = 30
    MIN_TRACK_SECONDS = 2  # shorter remainders of a sound track are dropped: the encoder pools by four frames

    def _audio_limits(self) -> Tuple[int, int]:
        proc = self.processor
        sr = int(getattr(proc, "sampling_rate", 16000) or 16000)
        seconds = int(getattr(proc, "audio_max_length", None) or (getattr(proc, "kwargs", {}) or {}).get("audio_max_length")
                      or self.DEFAULT_MAX_AUDIO_SECONDS)
        return sr, seconds * sr

    def sound_track(self, video_url: dict, data_folder: Optional[str], sr: int) -> Optional[np.ndarray]:
        """Sound track of a video: an explicit ``audio`` entry of the ``video_url`` dict, else a file with the
        video's name and a ``.wav`` / ``.flac`` / ``.mp3`` suffix next to it; ``None`` when there is none."""
        if video_url.get("audio"):
            return self.load_audio(video_url["audio"], sr=sr, data_folder=data_folder)[0]
        full = self._resolve(video_url["url"], data_folder)
        stem = os.path.splitext(full)[0]
        for suffix in (".wav", ".flac", ".mp3"):
            if os.path.exists(stem + suffix):
                return self.load_audio(stem + suffix, sr=sr)[0]
        return None

    def process_record(self, record: dict, data_folder: Optional[str] = "") -> Dict[str, torch.Tensor]:
        messages = copy.deepcopy(self.messages_of(record))
        sr, max_samples = self._audio_limits()
        want_track = bool((self.config.extra_kwargs or {}).get("use_audio_in_video", False))
        images, videos, audios, fps = [], [], [], []
        av = False
        for m in messages:
            content = m["content"] if isinstance(m["content"], list) else []
            new_content: List[dict] = []
            for c in content:
                t = c.get("type")
                if t == "image_url":
                    images.append(self.load_image(c["image_url"]["url"], data_folder))
                    new_content.append(c)
                elif t == "audio_url":
                    if c["audio_url"].get("url") == "from_video":
                        continue  # a placeholder written by an earlier pass over this record
                    wav = self.load_audio(c["audio_url"]["url"], sr=sr, data_folder=data_folder)[0]
                    for lo in range(0, max(len(wav), 1), max_samples):
                        audios.append(wav[lo:lo + max_samples])
                        new_content.append(c)  # one placeholder per chunk
                elif t == "video_url":
                    v = c["video_url"]
                    frames, f = self.load_video(v["url"], data_folder, v.get("video_start"), v.get("video_end"))
                    videos.append(frames)
                    fps.append(f)
                    track = self.sound_track(v, data_folder, sr) if want_track else None
                    if track is not None and len(track) >= self.MIN_TRACK_SECONDS * sr:
                        # the processor interleaves ONE audio clip with the video: keep the first chunk that fits
                        audios.append(track[:max_samples])
                        av = True
                    elif want_track:
                        logger.warning(f"use_audio_in_video: no usable sound track for {v['url']}")
                    new_content.append(c)
                else:
                    new_content.append(c)
            m["content"] = new_content
        if want_track and av and not all_videos_have_tracks(messages, videos, audios):
            av = False
        hf_messages = TrainUtilities.convert_open_to_hf(messages)
        out = self.processor.process(hf_messages, images=images or None, videos=videos or None, audios=audios or None,
                                     video_fps=fps or None, use_audio_in_video=av, sampling_rate=sr)
        return _truncate(self.config, out)


def all_videos_have_tracks(messages, videos, audios) -> bool:
    """The interleaved layout is all-or-nothing per record (as in the upstream processor): it needs one sound
    track per video."""
    n_audio_items = sum(1 for m in messages for c in (m["content"] if isinstance(m["content"], list) else []) if c.get("type") == "audio_url")
    return len(audios) - n_audio_items == len(videos)


# ------------------------------------------------------------------------------------------------ LLaVA-Video
class LlavaVideoRecords:
    """Time-aware videos, frame directories, CSV rows, time instructions."""

    @staticmethod
    def time_instruction(video_time: float, num_frames: int, frame_time: str) -> str:
        return (f"The video lasts for {video_time:.2f} seconds, and {num_frames} frames are uniformly sampled from it. "
                f"These frames are located at {frame_time}. Please answer the following questions related to this video.")

    def load_video_with_time(self, path: str, data_folder: Optional[str]) -> Tuple[Optional[np.ndarray], Optional[dict]]:
        kw = self.config.extra_kwargs or {}
        upbound = int(kw.get("frames_upbound", 0) or 0)
        force = bool(kw.get("force_sample", False))
        full = self._resolve(path, data_folder)
        try:
            if os.path.isdir(full):
                frames, meta = self._frames_from_directory(full)
            else:
                frames, meta = self.load_video_with_metadata(path, data_folder)
        except Exception as e:  # a damaged file skips the sample instead of ending the epoch
            logger.warning(f"could not decode {full}: {type(e).__name__}: {e}")
            return None, None
        times = list(meta["frame_times"])
        if upbound > 0 and (len(times) > upbound or force):
            keep = np.linspace(0, len(times) - 1, min(upbound, len(times)) if not force else upbound).round().astype(int)
            frames = frames[keep]
            times = [times[i] for i in keep]
        meta = dict(meta, frame_times=times, num_frames=len(times), frame_time=",".join(f"{t:.2f}s" for t in times),
                    sample_fps=len(times) / max(meta["video_time"], 1e-6))
        return frames, meta

    def _frames_from_directory(self, folder: str) -> Tuple[np.ndarray, dict]:
        """A directory of numbered frame images (the layout of ShareGPTVideo / LLaVA-Hound), taken to be one frame per
        second unless ``extra_kwargs.frame_dir_fps`` says otherwise; sampled at ``config.fps``."""
        from PIL import Image

        names = sorted(n for n in os.listdir(folder) if n.lower().endswith(IMAGE_SUFFIXES))
        if not names:
            raise FileNotFoundError(f"no frame images in {folder}")
        src_fps = float((self.config.extra_kwargs or {}).get("frame_dir_fps", 1.0))
        step = max(int(round(src_fps / max(float(self.config.fps or 1), 1e-6))), 1)
        idx = list(range(0, len(names), step))
        frames = np.stack([np.asarray(Image.open(os.path.join(folder, names[i])).convert("RGB")) for i in idx])
        times = [i / src_fps for i in idx]
        return frames, {"video_time": len(names) / src_fps, "frame_times": times, "fps": src_fps, "frames_indices": idx,
                        "total_num_frames": len(names), "sample_fps": len(idx) / max(len(names) / src_fps, 1e-6)}

    def messages_of(self, record: dict) -> List[dict]:
        if "messages" not in record and "video" in record and "prompt" in record:  # a CSV row
            msgs = [{"role": "user", "content": [{"type": "video_url", "video_url": {"url": record["video"]}},
                                                 {"type": "text", "text": str(record["prompt"])}]}]
            if record.get("answer") not in (None, ""):
                msgs.append({"role": "assistant", "content": [{"type": "text", "text": str(record["answer"])}]})
            return msgs
        return super().messages_of(record)

    def process_record(self, record: dict, data_folder: Optional[str] = "") -> Dict[str, torch.Tensor]:
        messages = copy.deepcopy(self.messages_of(record))
        kw = self.config.extra_kwargs or {}
        images, videos, fps, meta_first = [], [], [], None
        for m in messages:
            for c in (m["content"] if isinstance(m["content"], list) else []):
                if c.get("type") == "image_url":
                    images.append(self.load_image(c["image_url"]["url"], data_folder))
                elif c.get("type") == "video_url":
                    frames, meta = self.load_video_with_time(c["video_url"]["url"], data_folder)
                    if frames is None:
                        raise RuntimeError(f"unreadable video {c['video_url']['url']}")  # the caller skips the record
                    videos.append(frames)
                    fps.append(meta["sample_fps"])
                    meta_first = meta_first or meta
        if kw.get("add_time_instruction") and meta_first is not None:
            text = self.time_instruction(meta_first["video_time"], meta_first["num_frames"], meta_first["frame_time"])
            for m in messages:
                if m.get("role") == "user":
                    content = m["content"] if isinstance(m["content"], list) else [{"type": "text", "text": str(m["content"])}]
                    at = next((i for i, c in enumerate(content) if c.get("type") == "text"), len(content))
                    m["content"] = content[:at] + [{"type": "text", "text": text + "\n"}] + content[at:]
                    break
        pooling = {k: kw[k] for k in ("faster_token_stride", "mm_spatial_pool_stride", "mm_spatial_pool_mode") if k in kw}
        hf_messages = TrainUtilities.convert_open_to_hf(messages)
        out = self.processor.process(hf_messages, images=images or None, videos=videos or None, video_fps=fps or None, **pooling)
        return _truncate(self.config, out)


# ------------------------------------------------------------------------------------------------ registration
def _register(name: str, bases: tuple, doc: str):
    cls = type("".join(w.title() for w in name.split("_")) + "Dataset", bases, {"__doc__": doc, "__module__": __name__})
    register_dataset(name)(cls)
    return cls


Qwen3VLDataset = _register("qwen3_vl", (Qwen3VLRecords, MultiModalDataset), "Map-style Qwen3-VL dataset (videos with frame times).")
Qwen3VLIterableDataset = _register("qwen3_vl_iterable", (Qwen3VLRecords, MultiModalIterableDataset), "Streaming Qwen3-VL dataset.")
QwenOmniDataset = _register("qwen_omni", (QwenOmniRecords, MultiModalDataset), "Map-style Qwen-Omni dataset (audio chunks, sound tracks).")
QwenOmniIterableDataset = _register("qwen_omni_iterable", (QwenOmniRecords, MultiModalIterableDataset), "Streaming Qwen-Omni dataset.")
LlavaVideoDataset = _register("llava_video", (LlavaVideoRecords, MultiModalDataset), "LLaVA-Video dataset (time-aware videos).")
