"""Data plane of the realtime (streaming audio + video) model: processor ``aero_realtime``, dataset
``aero_realtime_iterable`` and their collator.

Token layout.  Audio is a timeline of ``<|audio_pad|>`` slots, one per ``2 * downsample_factor`` mel hops of 10 ms
(80 ms by default), between ``<|audio_start|>`` and ``<|audio_end|>``.  A parallel **text stream**
(``text_stream_ids``) mirrors ``input_ids`` except on those slots, where it carries ``<|rt_pad|>`` (silence) or the
tokens the assistant speaks at that moment; the model adds the audio rows to the text-stream embeddings.

* audio only: one envelope per clip, ``<|audio_start|> pad x N <|audio_end|>``;
* video with its sound track: the video is cut at its temporal patches and every patch becomes an envelope pair
  ``<t seconds> <|vision_start|> video_pad x S <|vision_end|> <|audio_start|> audio_pad x N_t <|audio_end|>`` where the
  ``N_t`` slots are the slots of the track whose time falls between this patch's time stamp and the next one's; text
  a user types at a given time is written in front of the first patch at or after that time;
* realtime supervision: every slot is a target (``<|rt_pad|>`` unless masked by ``rt_pad_label_mask_ratio``); an
  assistant segment that starts at time ``t`` takes the free slots from the first slot at or after ``t``: the first
  keeps ``<|rt_pad|>`` and is not supervised (the model is not asked to decide to start exactly there), the following
  carry the speech tokens in the stream and in the labels.  Nothing outside the slots is supervised;
* question answering over a video with a track and no timed segments: each (question, answer) pair is appended inside
  the user turn as ``question <|audio_start|> pad x n <|audio_end|>`` with ``n`` the number of answer tokens; the stream
  carries the answer in those slots, the labels supervise it, and ``n`` slots of silence are appended to the audio
  features so that every slot has its audio row.

Reference: src/lmms_engine/models/aero_realtime/processing_aero_realtime.py:197-830,
src/lmms_engine/datasets/processor/aero_realtime_processor.py:147-900,
src/lmms_engine/datasets/iterable/aero_realtime_iterable_dataset.py:51-330,
src/lmms_engine/datasets/collator/aero_realtime_collator.py.
"""
from __future__ import annotations

import os
from typing import Any, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..mapping_func import register_dataset, register_processor
from ..utils.logging_utils import logger
from .iterable.multimodal_iterable_dataset import MultiModalIterableDataset
from .processor.chat import IGNORE, Qwen3VLProcessor

MEDIA = ("image", "image_url", "video", "video_url", "audio", "audio_url")


def split_slots_over_chunks(n_slots: int, chunk_times: Sequence[float], slots_per_second: float) -> List[int]:
    """How many of ``n_slots`` audio slots belong to every video chunk: slot ``a`` lives at ``a / slots_per_second``
    seconds and belongs to the last chunk whose time stamp is not after it (the first chunk takes what precedes it)."""
    counts = [0] * len(chunk_times)
    if not counts or n_slots <= 0 or slots_per_second <= 0:
        return counts
    bounds = np.asarray(chunk_times[1:], dtype=np.float64)
    at = np.arange(n_slots, dtype=np.float64) / slots_per_second
    for c in np.searchsorted(bounds, at, side="right"):
        counts[int(c)] += 1
    return counts


def first_at_or_after(values: Sequence[float], target: float) -> int:
    for i, v in enumerate(values):
        if v >= target:
            return i
    return len(values)


def split_question_answers(messages) -> Tuple[List[Tuple[str, str]], List[dict]]:
    """``[(question, answer), ...]`` and the messages reduced to their media: the text of the user turns up to an
    assistant turn is that turn's question."""
    pairs, media_only, pending = [], [], []
    for m in messages:
        content = m["content"] if isinstance(m["content"], list) else [{"type": "text", "text": m["content"]}]
        if m["role"] == "system":
            media_only.append(m)
        elif m["role"] == "user":
            media = [c for c in content if c.get("type") in MEDIA]
            if media:
                media_only.append({"role": "user", "content": media})
            pending += [c["text"] for c in content if c.get("type") == "text" and c.get("text")]
        elif m["role"] == "assistant":
            said = [c["text"] for c in content if c.get("type") == "text" and c.get("text")]
            if said:
                pairs.append(("\n".join(pending).strip(), "\n".join(said)))
                pending = []
    return pairs, media_only


@register_processor("aero_realtime")
class AeroRealtimeProcessor(Qwen3VLProcessor):
    """``input_ids`` / ``text_stream_ids`` / ``labels`` (+ vision and audio tensors) of the realtime design.

    ``extra_kwargs``: ``num_mel_bins`` (128), ``max_frames`` (mel frames kept per clip, 3000), ``downsample_factor`` (4),
    ``rt_pad_label_mask_ratio`` (0), ``chunk_audio`` (false: clips stay ``[clips, mel, frames]``; true: the features
    are cut into one ``[mel, 2 * downsample_factor]`` piece per slot, encoded independently of each other),
    ``patch_size`` / ``min_pixels`` / ``max_pixels`` of the vision side, ``seed``."""

    def build(self):
        super().build()
        t, kw = self.tokenizer, self.kwargs
        names = ("<|audio_pad|>", "<|audio_start|>", "<|audio_end|>", "<|rt_pad|>")
        ids = {name: t.convert_tokens_to_ids(name) for name in names}
        missing = [k for k, v in ids.items() if v is None]
        if missing:
            raise ValueError(f"tokenizer lacks the realtime tokens {missing} (use a realtime checkpoint's tokenizer or 'byte_realtime')")
        self.audio_token_id, self.audio_start, self.audio_end, self.rt_pad = (ids[k] for k in names)
        self.n_mels = int(kw.get("num_mel_bins", 128))
        self.max_frames = int(kw.get("max_frames", 3000))
        self.df = int(kw.get("downsample_factor", 4))
        self.patch_size = int(kw.get("patch_size", self.patch_size))
        self.pad_mask_ratio = float(kw.get("rt_pad_label_mask_ratio", 0.0))
        self.chunk_audio = bool(kw.get("chunk_audio", False))
        self.rng = np.random.default_rng(int(kw.get("seed", 0)))
        self._rt: Dict[str, Any] = {}
        return self

    @property
    def mel_per_slot(self) -> int:
        return 2 * self.df

    @property
    def seconds_per_slot(self) -> float:
        return self.mel_per_slot * 160 / 16000.0

    # ---- entry point -------------------------------------------------------------------------------------------
    def process(self, hf_messages=None, images=None, videos=None, audios=None, add_system_prompt: bool = True,
                realtime_segments=None, video_fps=None, video_metadata=None, **kw):
        from .processor.audio_process import log_mel_spectrogram

        feats, masks, slots = [], [], []
        for wav in audios or []:
            f, m, valid = log_mel_spectrogram(wav, self.n_mels, self.max_frames)
            feats.append(f), masks.append(m)
            slots.append(max(valid // self.mel_per_slot, 1))
        self._rt = {"slots": slots, "segments": realtime_segments, "tails": [], "n_videos": len(videos or [])}
        try:
            if videos or images:
                out = super().process(hf_messages, images=images, videos=videos, audios=None, add_system_prompt=add_system_prompt,
                                      video_fps=video_fps, video_metadata=video_metadata)
            else:
                out = dict(self.build_ids_and_labels(hf_messages, {"image": [], "video": [], "audio": slots}, add_system_prompt))
            tails = self._rt["tails"]
        finally:
            self._rt = {}
        if feats or tails:
            out.update(self.audio_tensors(feats, masks, tails))
        return out

    def audio_tensors(self, feats, masks, tails: Sequence[int]) -> Dict[str, torch.Tensor]:
        """Clips (and one clip of silence per question-answer tail) as ``input_features`` + ``feature_attention_mask``."""
        per = self.mel_per_slot
        for n in tails:
            feats.append(torch.zeros(self.n_mels, n * per))
            masks.append(torch.ones(n * per, dtype=torch.long))
        if self.chunk_audio:
            rows, valid = [], []
            for f, m in zip(feats, masks):
                n = max(int(m.sum()) // per, 1)
                f = torch.nn.functional.pad(f, (0, max(n * per - f.shape[-1], 0)))[..., :n * per]
                rows.append(f.reshape(self.n_mels, n, per).permute(1, 0, 2))
                valid.append(torch.ones(n, per // 2, dtype=torch.long))
            return {"input_features": torch.cat(rows), "feature_attention_mask": torch.cat(valid)}
        longest = max(int(m.sum()) for m in masks)
        longest += longest % 2
        pad = lambda x: torch.nn.functional.pad(x, (0, max(longest - x.shape[-1], 0)))[..., :longest]  # noqa: E731
        return {"input_features": torch.stack([pad(f) for f in feats]), "feature_attention_mask": torch.stack([pad(m) for m in masks])}

    # ---- token streams -----------------------------------------------------------------------------------------
    def build_ids_and_labels(self, messages, mm, add_system_prompt=True) -> Dict[str, torch.Tensor]:
        rt = self._rt
        mm = dict(mm, audio=rt.get("slots", mm.get("audio", [])))
        if rt.get("n_videos") and mm["audio"]:
            return self._audio_video_streams(messages, mm, add_system_prompt)
        built = super().build_ids_and_labels(messages, mm, add_system_prompt)
        ids, labels = built["input_ids"], built["labels"]
        stream = ids.clone()
        positions = torch.nonzero(ids == self.audio_token_id, as_tuple=False).flatten().tolist()
        for pos in positions:
            stream[pos] = labels[pos] = self.rt_pad
        times = [k * self.seconds_per_slot for k in range(len(positions))]
        self._place_speech(positions, times, rt.get("segments"), stream, labels)
        self._mask_silence(labels)
        return {"input_ids": ids, "labels": labels, "text_stream_ids": stream}

    def _place_speech(self, positions, times, segments, stream, labels):
        taken = set()
        spoken = sorted((s for s in (segments or []) if s.get("role") == "assistant" and s.get("text")), key=lambda s: float(s["time"]))
        for seg in spoken:
            first = first_at_or_after(times, float(seg["time"]))
            free = [k for k in range(first, len(positions)) if k not in taken]
            if len(free) < 2:
                continue
            head = positions[free[0]]
            stream[head], labels[head] = self.rt_pad, IGNORE
            taken.add(free[0])
            for k, tok in zip(free[1:], self._enc(seg["text"])):
                stream[positions[k]] = labels[positions[k]] = tok
                taken.add(k)

    def _mask_silence(self, labels):
        if self.pad_mask_ratio > 0:
            silent = torch.nonzero(labels == self.rt_pad, as_tuple=False).flatten()
            drop = torch.from_numpy(self.rng.random(silent.numel()) < self.pad_mask_ratio)
            labels[silent[drop]] = IGNORE

    def chunk_times(self, i: int, grid_t: int) -> List[float]:
        """Time stamp of every temporal patch of video ``i``: the mean time of the frames merged into it."""
        times = self._video_times[i] if i < len(self._video_times) else None
        fps = float((self._video_fps[i] if i < len(self._video_fps) else None) or getattr(self.config, "fps", 1) or 1)
        tp, out = self.temporal_patch_size, []
        for f in range(grid_t):
            if times:
                group = [times[min(f * tp + j, len(times) - 1)] for j in range(tp)]
                out.append(sum(group) / len(group))
            else:
                out.append((f * tp + (tp - 1) / 2.0) / fps)
        return out

    def _audio_video_streams(self, messages, mm, add_system_prompt):
        rt = self._rt
        segments, slots, grids = rt["segments"], mm["audio"], mm["video_grids"]
        if len(slots) < len(grids):
            raise ValueError(f"{len(grids)} videos but {len(slots)} sound tracks: the interleaved layout needs one track per video")
        if len(slots) > len(grids):
            raise ValueError("audio clips next to videos with sound tracks are not part of the interleaved layout")
        pairs: List[Tuple[str, str]] = []
        if segments is None:
            pairs, base = split_question_answers(messages)
            base = base if pairs else messages
        else:
            media = [c for m in messages if m["role"] != "system" for c in (m["content"] if isinstance(m["content"], list) else [])
                     if c.get("type") in MEDIA]
            base = [m for m in messages if m["role"] == "system"] + [{"role": "user", "content": media}]
        typed = sorted((s for s in (segments or []) if s.get("role") == "user" and s.get("text")), key=lambda s: float(s["time"]))
        if add_system_prompt and (not base or base[0]["role"] != "system"):
            base = [{"role": "system", "content": self.default_system}] + list(base)
        unit = self.merge_size ** 2
        ids: List[int] = []
        slot_times: List[float] = []
        counters = {"image": 0, "video": 0}
        for m in base:
            ids += self._enc(f"<|im_start|>{m['role']}\n")
            content = m["content"] if isinstance(m["content"], list) else [{"type": "text", "text": m["content"]}]
            for c in content:
                kind = c.get("type")
                if kind == "text":
                    ids += self._enc(c["text"])
                elif kind in ("image", "image_url"):
                    ids += [self.vision_start] + [self.image_token_id] * mm["image"][counters["image"]] + [self.vision_end]
                    counters["image"] += 1
                elif kind in ("video", "video_url"):
                    v = counters["video"]
                    counters["video"] += 1
                    t, h, w = grids[v]
                    stamps = self.chunk_times(v, t)
                    duration = slots[v] * self.seconds_per_slot
                    per_chunk = split_slots_over_chunks(slots[v], stamps, slots[v] / duration if duration > 0 else 0.0)
                    typed_at = [[] for _ in range(t)]
                    for seg in typed:
                        typed_at[min(first_at_or_after(stamps, float(seg["time"])), t - 1)].append(seg["text"])
                    for f in range(t):
                        for text in typed_at[f]:
                            ids += self._enc(text)
                        ids += self._enc(f"<{stamps[f]:.1f} seconds>")
                        ids += [self.vision_start] + [self.video_token_id] * ((h * w) // unit) + [self.vision_end]
                        ids += [self.audio_start] + [self.audio_token_id] * per_chunk[f] + [self.audio_end]
                        slot_times += [stamps[f]] * per_chunk[f]
                    typed = []  # typed text belongs to the first video of the record
                # audio items have no placeholder of their own here: the track is inside the video envelopes
            ids += [self.im_end] + self._enc("\n")
        stream, labels = list(ids), [IGNORE] * len(ids)
        positions = [i for i, tok in enumerate(ids) if tok == self.audio_token_id]
        for pos in positions:
            stream[pos] = labels[pos] = self.rt_pad
        self._place_speech(positions, slot_times, segments, stream, labels)
        if pairs:
            closing = [self.im_end] + self._enc("\n")
            ids, stream, labels = (x[:-len(closing)] for x in (ids, stream, labels))
            for question, answer in pairs:
                q, a = (self._enc(question) if question else []), self._enc(answer)
                if not a:
                    continue
                ids += q + [self.audio_start] + [self.audio_token_id] * len(a) + [self.audio_end]
                stream += q + [self.audio_start] + a + [self.audio_end]
                labels += [IGNORE] * (len(q) + 1) + a + [IGNORE]
                rt["tails"].append(len(a))
            ids, stream, labels = ids + closing, stream + closing, labels + [IGNORE] * len(closing)
        labels_t = torch.tensor(labels, dtype=torch.long)
        self._mask_silence(labels_t)
        return {"input_ids": torch.tensor(ids, dtype=torch.long), "labels": labels_t,
                "text_stream_ids": torch.tensor(stream, dtype=torch.long)}

    def render_message(self, msg, counters, mm):
        """ChatML turn of the layouts without a sound track inside a video: audio clips are wrapped in their start /
        end markers, videos are written patch by patch with their time stamps."""
        ids = self._enc(f"<|im_start|>{msg['role']}\n")
        content = msg["content"] if isinstance(msg["content"], list) else [{"type": "text", "text": msg["content"]}]
        for c in content:
            kind = c.get("type")
            if kind == "text":
                ids += self._enc(c["text"])
            elif kind in ("audio", "audio_url"):
                n = mm["audio"][counters["audio"]]
                counters["audio"] += 1
                ids += [self.audio_start] + [self.audio_token_id] * n + [self.audio_end]
            elif kind in ("image", "image_url"):
                ids += [self.vision_start] + [self.image_token_id] * mm["image"][counters["image"]] + [self.vision_end]
                counters["image"] += 1
            elif kind in ("video", "video_url"):
                ids += self.render_video(counters, mm)
            else:
                raise ValueError(f"the realtime processor takes text, image, video and audio content, got {kind}")
        return ids + [self.im_end] + self._enc("\n")


class RealtimeCollator:
    """Packed collator that also concatenates the text stream along the token axis and pads the clips of all
    samples to one mel length."""

    def __call__(self, batch):
        from .collator.packed_collator import PackedCollator, _flatten

        samples = _flatten(batch)
        clips = [s for s in samples if "input_features" in s]
        width = max((s["input_features"].shape[-1] for s in clips), default=0)
        mask_width = max((s["feature_attention_mask"].shape[-1] for s in clips), default=0)
        padded = []
        for s in samples:
            s = dict(s)
            if "input_features" in s:
                s["input_features"] = torch.nn.functional.pad(s["input_features"], (0, width - s["input_features"].shape[-1]))
                s["feature_attention_mask"] = torch.nn.functional.pad(
                    s["feature_attention_mask"], (0, mask_width - s["feature_attention_mask"].shape[-1]))
            padded.append(s)
        return PackedCollator()(padded)


def mix_onto_track(track: np.ndarray, clip: np.ndarray, start_seconds: float, sr: int) -> np.ndarray:
    """``track`` with ``clip`` added from ``start_seconds`` on (the track grows when the clip runs past its end);
    the sum is scaled back into [-1, 1] when it clips."""
    lo = max(int(round(start_seconds * sr)), 0)
    out = np.zeros(max(len(track), lo + len(clip)), dtype=np.float32)
    out[:len(track)] = track
    out[lo:lo + len(clip)] += clip
    peak = float(np.abs(out).max()) if out.size else 0.0
    return out / peak if peak > 1.0 else out


@register_dataset("aero_realtime_iterable")
class AeroRealtimeIterableDataset(MultiModalIterableDataset):
    """``dataset_type: aero_realtime_iterable``.

    Timed speech comes from any of: a ``realtime_segments`` list of the record (``{"role", "time", "text"}``),
    ``{"type": "realtime_text", "start_sec", "text"}`` content items of assistant messages, or - when the record says
    ``"realtime": true`` - whole messages that carry a ``time``.  A video brings its sound track: the ``audio`` entry
    of its ``video_url`` dict, or a ``.wav`` / ``.flac`` / ``.mp3`` file of the same name next to it (a video without one
    is processed as frames only).  ``user_audio`` entries (``{"path", "start_time"}``) are mixed onto the first track:
    spoken questions."""

    TRACK_SUFFIXES = (".wav", ".flac", ".mp3")

    def sound_track(self, video_url: dict, data_folder, sr: int) -> Optional[np.ndarray]:
        if video_url.get("audio"):
            track = self.load_audio(video_url["audio"], sr=sr, data_folder=data_folder)[0]
        else:
            stem = os.path.splitext(self._resolve(video_url["url"], data_folder))[0]
            found = next((stem + s for s in self.TRACK_SUFFIXES if os.path.exists(stem + s)), None)
            if found is None:
                return None
            track = self.load_audio(found, sr=sr)[0]
        lo = float(video_url.get("video_start") or 0.0)
        hi = video_url.get("video_end")
        return track[int(lo * sr): int(float(hi) * sr) if hi is not None else None]

    def process_record(self, record: dict, data_folder=""):
        from ..utils.train_utils import TrainUtilities

        sr = 16000
        segments = [dict(s) for s in (record.get("realtime_segments") or [])]
        realtime = bool(record.get("realtime", False))
        images, videos, audios, metadata, kept = [], [], [], [], []
        for m in self.messages_of(record):
            content = m["content"] if isinstance(m["content"], list) else [{"type": "text", "text": m["content"]}]
            if realtime and m.get("time") is not None and m["role"] in ("user", "assistant"):
                text = "\n".join(c["text"] for c in content if c.get("type") == "text" and c.get("text"))
                if text:
                    segments.append({"time": float(m["time"]), "role": m["role"], "text": text})
                continue
            new_content = []
            for c in content:
                kind = c.get("type")
                if kind == "realtime_text":
                    segments.append({"time": float(c["start_sec"]), "role": "assistant", "text": c["text"]})
                    continue
                if kind == "image_url":
                    images.append(self.load_image(c["image_url"]["url"], data_folder))
                elif kind == "audio_url":
                    audios.append(self.load_audio(c["audio_url"]["url"], sr=sr, data_folder=data_folder)[0])
                elif kind == "video_url":
                    v = c["video_url"]
                    frames, meta = self.load_video_with_metadata(v["url"], data_folder, v.get("video_start"), v.get("video_end"))
                    start = float(v.get("video_start") or 0.0)
                    meta = dict(meta, frame_times=[t - start for t in meta["frame_times"]])
                    track = self.sound_track(v, data_folder, sr)
                    if track is None:
                        logger.warning(f"no sound track for {v['url']}: processed as frames only")
                    else:
                        audios.append(track)
                    videos.append(frames), metadata.append(meta)
                new_content.append(c)
            kept.append({"role": m["role"], "content": new_content})
        for entry in record.get("user_audio") or []:
            if not audios:
                raise ValueError("user_audio needs a sound track to be mixed onto")
            clip = self.load_audio(entry["path"], sr=sr, data_folder=data_folder)[0]
            audios[0] = mix_onto_track(audios[0], clip, float(entry.get("start_time", 0.0)), sr)
        hf_messages = TrainUtilities.convert_open_to_hf(kept)
        out = self.processor.process(hf_messages, images=images or None, videos=videos or None, audios=audios or None,
                                     realtime_segments=segments or None, video_metadata=metadata or None)
        limit = self.config.max_length
        if limit and out["input_ids"].numel() > limit:
            raise ValueError(f"realtime sample of {out['input_ids'].numel()} tokens exceeds max_length={limit}: the audio rows "
                             f"would no longer match their slots")
        return out

    def get_collator(self):
        return RealtimeCollator()
