"""Datasets and processors of the non-chat trainers and of plain-text pre-training.

* ``fineweb_edu`` (iterable): rows with a ``text`` field, every token supervised, packed online
  (reference: src/lmms_engine/datasets/iterable/fineweb_edu_dataset.py).
* ``sit`` (map-style): pre-computed latents + class labels for the SiT trainer
  (reference: src/lmms_engine/datasets/naive/sit_dataset.py).
* ``rae`` (map-style): images resized to a fixed square for the autoencoder / discriminator trainer
  (reference: src/lmms_engine/datasets/naive/rae_dataset.py).
* ``bagel_iterable`` + processor ``bagel``: interleaved text / image conversations for the unified
  understanding + generation model: every text span is ``<|im_start|> ids <|im_end|>`` (assistant spans
  supervised), every image is ``<|vision_start|> latent tokens <|vision_end|>`` sharing one rotary position;
  assistant images are generation targets (random noise level), user images are clean conditions
  (reference: src/lmms_engine/datasets/processor/bagel_processor.py:91-365, collator/bagel_collator.py:11-80).
* processors ``sit``, ``rae_siglip``, ``wanvideo`` (tensor normalisation only) and ``nanovlm`` (ChatML text
  plus NaFlex patches: an image is resized so that it has at most ``max_num_patches`` patches of
  ``patch_size`` pixels and is flattened to ``[rows*cols, C*p*p]`` with its ``spatial_shapes`` row).
"""
from __future__ import annotations

import math
import os
from typing import Any, Dict, List

import numpy as np
import torch
from torch.utils.data import Dataset

from ..mapping_func import register_dataset, register_processor
from .base import DatasetCore
from .iterable.multimodal_iterable_dataset import MultiModalIterableDataset
from .processor.chat import ChatProcessor
from .synthetic import StackCollator


# ------------------------------------------------------------------------------- text pre-training
@register_dataset("fineweb_edu")
class FinewebEduDataset(MultiModalIterableDataset):
    """``{"text": ...}`` rows -> ``input_ids`` (+ end-of-text) with every token a target."""

    def process_record(self, record: dict, data_folder: str = "") -> Dict[str, torch.Tensor]:
        tok = self.processor.tokenizer
        ids = list(tok.encode(record["text"], add_special_tokens=False))
        eos = getattr(tok, "eos_token_id", None)
        if eos is not None:
            ids.append(int(eos))
        limit = self.config.max_length or self.config.packing_length
        if limit:
            ids = ids[: int(limit)]
        t = torch.tensor(ids, dtype=torch.long)
        return {"input_ids": t, "labels": t.clone()}


# ------------------------------------------------------------------------------- tensor processors
class TensorProcessor:
    """No tokenizer: scales / normalises tensors.  ``extra_kwargs``: ``mean``, ``std``, ``image_size``."""

    def __init__(self, config):
        self.config = config
        self.kwargs = dict(getattr(config, "extra_kwargs", {}) or {})
        self.mean = float(self.kwargs.get("mean", 0.5))
        self.std = float(self.kwargs.get("std", 0.5))
        self.image_size = int(self.kwargs.get("image_size", 256))

    def build(self):
        return self

    @property
    def processor(self):
        return self

    def save_pretrained(self, path: str):
        os.makedirs(path, exist_ok=True)

    def image_to_tensor(self, img) -> torch.Tensor:
        """PIL image / HWC uint8 array -> ``[3, S, S]`` float, centre-cropped, normalised."""
        from PIL import Image

        if not isinstance(img, Image.Image):
            img = Image.fromarray(np.asarray(img).astype(np.uint8))
        img = img.convert("RGB")
        w, h = img.size
        s = min(w, h)
        img = img.crop(((w - s) // 2, (h - s) // 2, (w - s) // 2 + s, (h - s) // 2 + s)).resize((self.image_size, self.image_size), Image.BICUBIC)
        x = torch.from_numpy(np.asarray(img).copy()).permute(2, 0, 1).float() / 255.0
        return (x - self.mean) / self.std

    def process(self, image=None, **kw):
        return {"pixel_values": self.image_to_tensor(image)} if image is not None else {}


register_processor("tensor")(TensorProcessor)  # family processors: datasets/processor/generative_processors.py


@register_processor("nanovlm")
class NanovlmProcessor(ChatProcessor):
    """ChatML text with one placeholder per image patch and NaFlex patch rows."""

    def build(self):
        super().build()
        self.patch = int(self.kwargs.get("patch_size", 16))
        self.max_patches = int(self.kwargs.get("max_num_patches", 256))
        return self

    def patchify(self, img):
        from PIL import Image

        img = img.convert("RGB") if isinstance(img, Image.Image) else Image.fromarray(np.asarray(img).astype(np.uint8)).convert("RGB")
        w, h = img.size
        p = self.patch
        scale = math.sqrt(self.max_patches * p * p / (w * h))
        rows = max(1, min(int(h * scale) // p, self.max_patches))
        cols = max(1, min(int(w * scale) // p, self.max_patches // rows))
        img = img.resize((cols * p, rows * p), Image.BILINEAR)
        x = torch.from_numpy(np.asarray(img).copy()).float() / 255.0  # [H, W, C]
        x = (x - 0.5) / 0.5
        x = x.view(rows, p, cols, p, 3).permute(0, 2, 4, 1, 3).reshape(rows * cols, 3 * p * p)
        return x, (rows, cols)

    def process(self, hf_messages=None, images=None, videos=None, audios=None, add_system_prompt: bool = True, **kw):
        out: Dict[str, torch.Tensor] = {}
        mm = {"image": [], "video": [], "audio": []}
        if images:
            pats, shapes = zip(*(self.patchify(im) for im in images))
            out["pixel_values"] = torch.cat(pats)
            out["spatial_shapes"] = torch.tensor(shapes, dtype=torch.long)
            mm["image"] = [r * c for r, c in shapes]
        out.update(self.build_ids_and_labels(hf_messages, mm, add_system_prompt))
        return out


@register_processor("aero")
@register_processor("qwen2_audio")
class Qwen2AudioProcessor(ChatProcessor):
    """ChatML text with ``<|AUDIO|>`` placeholders: one per pooled encoder frame of every audio clip."""

    def build(self):
        super().build()
        self.n_mels = int(self.kwargs.get("num_mel_bins", 128))
        self.n_frames = int(self.kwargs.get("max_frames", 3000))
        return self

    def process(self, hf_messages=None, images=None, videos=None, audios=None, add_system_prompt: bool = True, **kw):
        from .processor.audio_process import log_mel_spectrogram

        out: Dict[str, torch.Tensor] = {}
        mm = {"image": [], "video": [], "audio": []}
        if audios:
            feats, masks = [], []
            for wav in audios:
                f, m, valid = log_mel_spectrogram(wav, self.n_mels, self.n_frames)
                feats.append(f), masks.append(m)
                frames = (valid - 1) // 2 + 1  # after the stride-2 convolution
                mm["audio"].append(max((frames - 2) // 2 + 1, 1))  # after the average pooling by 2
            out["audio_values"] = torch.stack(feats)
            out["audio_attention_mask"] = torch.stack(masks)
        out.update(self.build_ids_and_labels(hf_messages, mm, add_system_prompt))
        return out


from .processor.chat import QwenVLProcessor  # noqa: E402


@register_processor("Qwen2_5OmniProcessor")
@register_processor("qwen2_5_omni")
class OmniProcessor(QwenVLProcessor):
    """Qwen2.5-VL image / video handling plus log-mel audio clips (one placeholder per pooled encoder row).
    Temporal positions of videos advance ``position_id_per_seconds`` (25) per second."""

    tokens_per_second = 25.0

    def build(self):
        super().build()
        self.n_mels = int(self.kwargs.get("num_mel_bins", 128))
        self.n_frames = int(self.kwargs.get("max_frames", 3000))
        self._audio_counts = []
        return self

    def build_ids_and_labels(self, messages, mm, add_system_prompt=True):
        mm = dict(mm, audio=list(self._audio_counts))
        self._mm_now = mm
        return super().build_ids_and_labels(messages, mm, add_system_prompt)

    # ---- a video that carries its sound track ("use_audio_in_video") ------------------------------------
    # The clip's audio placeholders are interleaved with its video placeholders in chunks of ``seconds_per_chunk``
    # seconds, between <|vision_start|><|audio_bos|> and <|audio_eos|><|vision_end|>; the audio clip of the video is
    # the next one in ``audios`` (datasets put it at the video's place in the list).
    seconds_per_chunk = 2.0
    use_audio_in_video = False

    def render_video(self, counters, mm) -> List[int]:
        if not self.use_audio_in_video:
            return super().render_video(counters, mm)
        from ..models.mrope import interleave_av

        i = counters["video"]
        counters["video"] += 1
        n_audio = mm["audio"][counters["audio"]]
        counters["audio"] += 1
        t, h, w = mm["video_grids"][i]
        per = (h // self.merge_size) * (w // self.merge_size)
        sec = self._second_per_grid[i] if i < len(self._second_per_grid) else 1.0
        vt = np.floor(np.repeat(np.arange(t), per) * sec * self.tokens_per_second).astype(np.int64)
        ids = [self.vision_start] + ([self.audio_bos] if self.audio_bos is not None else [])
        for kind, lo, hi in interleave_av(vt, n_audio, int(self.tokens_per_second * self.seconds_per_chunk)):
            ids += [self.video_token_id if kind == "video" else self.audio_token_id] * (hi - lo)
        ids += ([self.audio_eos] if self.audio_eos is not None else []) + [self.vision_end]
        return ids + self._enc("\n")

    def positions(self, out) -> torch.Tensor:
        if not self.use_audio_in_video:
            return super().positions(out)
        from ..models.mrope import omni_positions_one

        if self.audio_bos is None or self.audio_eos is None:
            raise ValueError("use_audio_in_video needs a tokenizer with <|audio_bos|> / <|audio_eos|>")
        img = out["image_grid_thw"].tolist() if "image_grid_thw" in out else []
        vid = out["video_grid_thw"].tolist() if "video_grid_thw" in out else []
        spg = out["second_per_grid_ts"].tolist() if "second_per_grid_ts" in out else None
        pos = omni_positions_one(out["input_ids"].numpy(), self.image_token_id, self.video_token_id, self.audio_token_id, img, vid, spg,
                                 self.merge_size, self.tokens_per_second, self.seconds_per_chunk)
        return torch.from_numpy(pos)

    def process(self, hf_messages=None, images=None, videos=None, audios=None, add_system_prompt: bool = True,
                use_audio_in_video: bool = False, **kw):
        from .processor.audio_process import log_mel_spectrogram

        tok = self.tokenizer
        self.audio_bos = self._maybe_token("<|audio_bos|>")
        self.audio_eos = self._maybe_token("<|audio_eos|>")
        self.use_audio_in_video = bool(use_audio_in_video) and bool(videos) and bool(audios)
        fps = kw.get("video_fps")
        self._second_per_grid = [self.temporal_patch_size / float((fps[i] if fps and i < len(fps) else None) or getattr(self.config, "fps", 1) or 1)
                                 for i in range(len(videos or []))]
        del tok
        audio_out, self._audio_counts = {}, []
        if audios:
            feats, masks = [], []
            for wav in audios:
                f, m, valid = log_mel_spectrogram(wav, self.n_mels, self.n_frames)
                feats.append(f), masks.append(m)
                after = (valid - 1) // 2 + 1
                self._audio_counts.append(max((after - 2) // 2 + 1, 1))
            audio_out = {"audio_values": torch.stack(feats), "audio_attention_mask": torch.stack(masks)}
        try:
            out = super().process(hf_messages, images=images, videos=videos, audios=None, add_system_prompt=add_system_prompt, **kw)
        finally:
            self._audio_counts = []
            self.use_audio_in_video = False
        out.update(audio_out)
        return out

    def _maybe_token(self, text: str):
        try:
            ix = self.tokenizer.convert_tokens_to_ids(text)
        except Exception:
            return None
        unk = getattr(self.tokenizer, "unk_token_id", None)
        return None if ix is None or (unk is not None and ix == unk) else int(ix)


from .processor.chat import Qwen3VLProcessor  # noqa: E402


@register_processor("Qwen3OmniMoeProcessor")
@register_processor("qwen3_omni_moe")
class Omni3Processor(Qwen3VLProcessor):
    """Qwen3-VL image / video handling plus log-mel audio clips; one placeholder per row of the Qwen3-Omni audio
    encoder (13 rows per 100 mel frames)."""

    build = OmniProcessor.build
    build_ids_and_labels = OmniProcessor.build_ids_and_labels

    def process(self, hf_messages=None, images=None, videos=None, audios=None, add_system_prompt: bool = True, **kw):
        from ..models.audio import omni3_output_lengths
        from .processor.audio_process import log_mel_spectrogram

        audio_out, self._audio_counts = {}, []
        if audios:
            feats, masks = [], []
            for wav in audios:
                f, m, valid = log_mel_spectrogram(wav, self.n_mels, self.n_frames)
                feats.append(f), masks.append(m)
                self._audio_counts.append(max(int(omni3_output_lengths(torch.tensor([valid]))[0]), 1))
            audio_out = {"audio_values": torch.stack(feats), "audio_attention_mask": torch.stack(masks)}
        try:
            out = Qwen3VLProcessor.process(self, hf_messages, images=images, videos=videos, audios=None,
                                           add_system_prompt=add_system_prompt, **kw)
        finally:
            self._audio_counts = []
        out.update(audio_out)
        return out


@register_processor("llava_video")
@register_processor("llava_onevision")
@register_processor("llava")
class LlavaOnevisionProcessor(ChatProcessor):
    """Any-resolution tiling of LLaVA-OneVision: an image becomes a resized base view plus the tiles of the
    best-fitting grid resolution (aspect-preserving resize, centred zero padding); the number of placeholders
    is what the model's packing of the tile features produces.  Video frames are resized to one tile each."""

    def build(self):
        super().build()
        kw = self.kwargs
        self.tile = int(kw.get("image_size", 384))
        self.patch = int(kw.get("patch_size", 14))
        self.max_tiles = int(str(kw.get("vision_aspect_ratio", "anyres_max_9")).replace("anyres_max_", ""))
        self.pinpoints = kw.get("image_grid_pinpoints") or [[self.tile * i, self.tile * j] for i in range(1, 7) for j in range(1, 7)]
        self.mean, self.std = float(kw.get("mean", 0.5)), float(kw.get("std", 0.5))
        return self

    def _to_tensor(self, img):
        x = torch.from_numpy(np.asarray(img.convert("RGB")).copy()).permute(2, 0, 1).float() / 255.0
        return (x - self.mean) / self.std

    def tiles_of(self, img):
        from PIL import Image

        from ..models.llava_ov import select_best_resolution

        img = img if isinstance(img, Image.Image) else Image.fromarray(np.asarray(img).astype(np.uint8))
        w, h = img.size
        bh, bw = select_best_resolution((h, w), [tuple(p) for p in self.pinpoints])
        scale = min(bw / w, bh / h)
        nw, nh = max(int(math.ceil(w * scale)), 1), max(int(math.ceil(h * scale)), 1)
        nw, nh = min(nw, bw), min(nh, bh)
        canvas = Image.new("RGB", (bw, bh), (0, 0, 0))
        canvas.paste(img.convert("RGB").resize((nw, nh), Image.BICUBIC), ((bw - nw) // 2, (bh - nh) // 2))
        t = self.tile
        tiles = [self._to_tensor(img.resize((t, t), Image.BICUBIC))]
        for i in range(0, bh, t):
            for j in range(0, bw, t):
                tiles.append(self._to_tensor(canvas.crop((j, i, j + t, i + t))))
        return torch.stack(tiles), (h, w)

    def process(self, hf_messages=None, images=None, videos=None, audios=None, add_system_prompt: bool = True, **kw):
        from PIL import Image

        from ..models.llava_ov import packed_image_tokens

        out: Dict[str, torch.Tensor] = {}
        mm = {"image": [], "video": [], "audio": []}
        side = self.tile // self.patch
        if images:
            tiles, sizes = zip(*(self.tiles_of(im) for im in images))
            out["pixel_values"] = torch.cat(tiles)  # tiles of all images, in order
            out["image_sizes"] = torch.tensor(sizes, dtype=torch.long)
            mm["image"] = [packed_image_tokens(s, self.pinpoints, self.tile, side, self.max_tiles) for s in sizes]
        if videos:
            clips = []
            for frames in videos:
                fr = [self._to_tensor(Image.fromarray(np.asarray(f).astype(np.uint8)).resize((self.tile, self.tile), Image.BICUBIC)) for f in frames]
                clips.append(torch.stack(fr))
                mm["video"].append(len(fr) * math.ceil(side / 2) ** 2 + 1)
            if len({c.shape[0] for c in clips}) == 1:
                out["pixel_values_videos"] = torch.stack(clips)
            else:
                raise ValueError("clips of one sample must have the same number of frames")
        out.update(self.build_ids_and_labels(hf_messages, mm, add_system_prompt))
        return out


# ------------------------------------------------------------------------------- map-style tensor datasets
class _RecordDataset(DatasetCore, Dataset):
    def __init__(self, config):
        super().__init__(config)

    def __len__(self):
        return len(self.data_list)

    def get_collator(self):
        return StackCollator()


@register_dataset("sit")
class SitDataset(_RecordDataset):
    """Rows ``{"latent": path (.pt / .npy) | nested list, "label": int}`` or ``{"image": path, "label": int}``."""

    def __getitem__(self, i) -> Dict[str, Any]:
        rec, folder = self.data_list[i], self.data_folder[i]
        if "image" in rec:
            return self.processor.process(image=self.load_image(os.path.join(folder or "", rec["image"])), label=rec.get("label", 0))
        lat = rec["latent"]
        if isinstance(lat, str):
            path = os.path.join(folder or "", lat)
            lat = torch.load(path, map_location="cpu") if path.endswith(".pt") else torch.from_numpy(np.load(path))
        return {"latents": torch.as_tensor(lat, dtype=torch.float32), "labels": torch.tensor(int(rec.get("label", 0)))}


@register_dataset("rae")
class RaeDataset(_RecordDataset):
    """Rows ``{"image": path}`` -> ``pixel_values [3, S, S]``."""

    def __getitem__(self, i) -> Dict[str, Any]:
        rec, folder = self.data_list[i], self.data_folder[i]
        img = self.load_image(os.path.join(folder or "", rec["image"]))
        return {"pixel_values": self.processor.image_to_tensor(img)}


# ------------------------------------------------------------------------------- unified understanding + generation
@register_processor("bagel")
class BagelProcessor(ChatProcessor):
    """Builds the packed stream of ``models/bagel.py`` from one conversation.

    Images arrive as latents ``[C, h, w]`` (precomputed with the VAE: ``.pt`` / ``.npy`` files, the way the video
    pipeline stores its latents) or, with ``latent_from_pixels: true``, as PIL images that are average-pooled by
    ``vae_downsample`` into 3-channel pseudo-latents.  ``latent_patch_size`` x ``latent_patch_size`` latent cells form
    one token.  Dropout of text / image conditions for classifier-free guidance follows the reference's
    probabilities (``text_cond_dropout_prob``, ``vae_cond_dropout_prob``)."""

    def build(self):
        super().build()
        kw = self.kwargs
        self.p = int(kw.get("latent_patch_size", 2))
        self.down = int(kw.get("vae_downsample", 8))
        self.max_latent = int(kw.get("max_latent_size", 64))
        self.from_pixels = bool(kw.get("latent_from_pixels", False))
        self.text_drop = float(kw.get("text_cond_dropout_prob", 0.0))
        self.vae_drop = float(kw.get("vae_cond_dropout_prob", 0.0))
        self.rng = np.random.default_rng(int(kw.get("seed", 0)))
        return self

    def to_latent(self, img) -> torch.Tensor:
        if torch.is_tensor(img):
            return img.float()
        if isinstance(img, np.ndarray) and img.ndim == 3 and img.dtype != np.uint8:
            return torch.from_numpy(img).float()
        if not self.from_pixels:
            raise ValueError("bagel processor: image is not a latent tensor; precompute latents or set latent_from_pixels")
        from PIL import Image

        img = img.convert("RGB") if isinstance(img, Image.Image) else Image.fromarray(np.asarray(img).astype(np.uint8)).convert("RGB")
        cell = self.down * self.p
        w, h = img.size
        side = self.max_latent * self.down
        scale = min(1.0, side / max(w, h))
        w, h = max(cell, int(w * scale) // cell * cell), max(cell, int(h * scale) // cell * cell)
        x = torch.from_numpy(np.asarray(img.resize((w, h), Image.BICUBIC)).copy()).float().permute(2, 0, 1) / 127.5 - 1.0
        return torch.nn.functional.avg_pool2d(x[None], self.down)[0]

    def latent_tokens(self, lat: torch.Tensor):
        """``[C, h, w]`` -> ``[h/p * w/p, C*p*p]`` tokens and their position ids on the ``max_latent`` grid."""
        C, h, w = lat.shape
        p = self.p
        rows, cols = h // p, w // p
        # inside a patch: (pixel row, pixel column, channel), the order of the released input / output projections
        tok = lat[:, : rows * p, : cols * p].reshape(C, rows, p, cols, p).permute(1, 3, 2, 4, 0).reshape(rows * cols, p * p * C)
        pos = (torch.arange(rows)[:, None] * self.max_latent + torch.arange(cols)[None, :]).flatten()
        return tok, pos

    def process(self, hf_messages=None, images=None, videos=None, audios=None, add_system_prompt: bool = True, **kw):
        ids: List[int] = []
        labels: List[int] = []
        pos: List[int] = []
        lat_tok, lat_pos, lat_idx, lat_t, lat_loss = [], [], [], [], []
        splits: List[List[int]] = []  # [length, mode]: 0 causal text, 1 full (clean image), 2 noise (noised target image)
        rope, image_at = 0, 0
        for msg in hf_messages:
            role = msg["role"]
            content = msg["content"] if isinstance(msg["content"], list) else [{"type": "text", "text": msg["content"]}]
            for c in content:
                kind = c.get("type")
                if kind == "text":
                    if role != "assistant" and self.text_drop > 0 and self.rng.random() < self.text_drop:
                        continue
                    body = self._enc(c["text"])
                    span = [self.im_start] + body + [self.im_end]
                    # the model shifts labels itself: a supervised position holds its own token
                    labels += ([-100] + body + [self.im_end]) if role == "assistant" else [-100] * len(span)
                    ids += span
                    pos += list(range(rope, rope + len(span)))
                    rope += len(span)
                    if splits and splits[-1][1] == 0:
                        splits[-1][0] += len(span)
                    else:
                        splits.append([len(span), 0])
                elif kind in ("image", "image_url"):
                    img = images[image_at]
                    image_at += 1
                    target = role == "assistant"
                    if not target and self.vae_drop > 0 and self.rng.random() < self.vae_drop:
                        rope += 1  # a dropped condition image still advances the position
                        continue
                    tok, tpos = self.latent_tokens(self.to_latent(img))
                    n = tok.shape[0]
                    start = len(ids) + 1
                    ids += [self.vision_start] + [self.image_token_id] * n + [self.vision_end]
                    labels += [-100] * (n + 2)
                    pos += [rope] * (n + 2)
                    rope += 1
                    lat_tok.append(tok)
                    lat_pos.append(tpos)
                    lat_idx.append(torch.arange(start, start + n))
                    # generation targets get a logit-normal noise level, condition images stay clean
                    t = float(1.0 / (1.0 + math.exp(-self.rng.standard_normal()))) if target else 0.0
                    lat_t.append(torch.full((n,), t))
                    lat_loss.append(torch.full((n,), target, dtype=torch.bool))
                    splits.append([n + 2, 2 if target else 1])
        out = {"input_ids": torch.tensor(ids, dtype=torch.long), "labels": torch.tensor(labels, dtype=torch.long),
               "position_ids": torch.tensor(pos, dtype=torch.long)}
        if self.kwargs.get("attention_modes", True) and splits:
            out["split_lens"] = torch.tensor([s[0] for s in splits], dtype=torch.long)
            out["attn_modes"] = torch.tensor([s[1] for s in splits], dtype=torch.long)
        if lat_tok:
            out.update(latent_tokens=torch.cat(lat_tok), latent_pos=torch.cat(lat_pos), latent_index=torch.cat(lat_idx),
                       timesteps=torch.cat(lat_t), latent_loss_mask=torch.cat(lat_loss))
        return out


class BagelCollator:
    """Packed stream over several conversations: like the packed collator, with every ``*_index`` tensor moved by
    the start of its conversation."""

    def __call__(self, batch):
        from .collator.packed_collator import PackedCollator, _flatten

        samples, at, moved = _flatten(batch), 0, []
        for s in samples:
            s = dict(s)
            for k in list(s):
                if k.endswith("_index") and torch.is_tensor(s[k]):
                    s[k] = s[k] + at
            at += int(s["input_ids"].numel())
            moved.append(s)
        return PackedCollator()(moved)


@register_dataset("bagel_iterable")
class BagelIterableDataset(MultiModalIterableDataset):
    """``dataset_type: bagel_iterable``: the vision iterable dataset whose images may be stored latents."""

    def load_image(self, url, data_folder=None):
        path = os.path.join(data_folder, url) if data_folder and not os.path.isabs(str(url)) else url
        if str(path).endswith(".pt"):
            return torch.load(path, map_location="cpu", weights_only=True)
        if str(path).endswith(".npy"):
            return torch.from_numpy(np.load(path))
        return super().load_image(url, data_folder)

    def get_collator(self):
        return BagelCollator()
