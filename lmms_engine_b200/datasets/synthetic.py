"""Synthetic packed-token datasets (no files, no tokenizer): documents with lengths uniform
in ``[min_len, max_len]`` and token ids uniform in ``[0, vocab)``, packed online into rows of
``packing_length`` tokens.  Used by the plumbing tests and by ``bench.py``; the reference's
tests download a real dataset instead (cicd/run_traincicd.sh:51-62)."""
from __future__ import annotations

from typing import Any, Dict, Iterator, List, Optional

import numpy as np
import torch
from torch.utils.data import IterableDataset

from ..mapping_func import register_dataset
from .collator.packed_collator import PackedCollator
from .packing import build_online_packer


@register_dataset("synthetic_packed")
class SyntheticPackedDataset(IterableDataset):
    """Yields packs: ``List[{"input_ids": LongTensor, "labels": LongTensor}]``.

    ``extra_kwargs`` of the dataset config: ``vocab_size`` (4096), ``min_len`` (32),
    ``max_len`` (512), ``num_documents`` (per rank, default unlimited), ``fill_exact``
    (truncate the last document of a pack so that every pack has exactly
    ``packing_length`` tokens).
    """

    def __init__(self, config):
        self.config = config
        kw = dict(config.extra_kwargs or {})
        self.vocab = int(kw.get("vocab_size", 4096))
        self.min_len = int(kw.get("min_len", 32))
        self.max_len = int(kw.get("max_len", 512))
        self.num_documents = kw.get("num_documents")
        self.fill_exact = bool(kw.get("fill_exact", False))
        self.pattern = kw.get("pattern", "uniform")  # "uniform" | "periodic" (learnable)
        self.interleave_ranks = int(kw.get("interleave_ranks", 0) or 0)
        self.prompt_len = int(kw.get("prompt_len", 0) or 0)
        self.collator_type = kw.get("collator_type", "packed")
        self.mask_token_id = int(kw.get("mask_token_id", self.vocab - 1))
        self.packing_length = int(config.packing_length or 1024)
        self.strategy = config.packing_strategy or "first_fit"
        self.packing_kwargs = dict(kw.get("packing_kwargs", {}) or {})
        self.seed = int(config.data_seed or 0)
        self.dp_rank, self.dp_size = 0, 1
        self.cur_idx = 0  # documents consumed (resume point)
        self.processor = None

    # -- reference dataset API -----------------------------------------------------------
    def build(self):
        try:
            from ..parallel import process_group_manager as pgm

            m = pgm.process_group_manager
            if m is not None:
                self.dp_rank, self.dp_size = m.dp_rank, m.dp_size
        except Exception:
            pass
        return self

    def get_collator(self):
        if self.collator_type == "dllm":
            from .collator.text_dllm_collator import TextDllmCollator

            return TextDllmCollator(self.mask_token_id, seed=self.seed)
        if self.collator_type == "padded":
            # [n_docs, max_len] with attention_mask: the layout models from the transformers library take
            from .collator.vision_collator import VisionCollator

            return VisionCollator(pad_token_id=0)
        return PackedCollator()

    def state_dict(self) -> Dict[str, Any]:
        return {"cur_idx": self.cur_idx}

    def load_state_dict(self, sd: Dict[str, Any]) -> None:
        self.cur_idx = int(sd.get("cur_idx", 0))

    def _document(self, idx: int) -> Dict[str, torch.Tensor]:
        # every document is a pure function of (seed, rank, index): resumable and reproducible
        rng = np.random.default_rng([self.seed, self.dp_rank, idx])
        n = int(rng.integers(self.min_len, self.max_len + 1))
        if self.pattern == "periodic":
            # a short random motif repeated: learnable, so tests can watch the loss fall
            period = int(rng.integers(2, 6))
            motif = rng.integers(0, min(self.vocab, 64), size=period, dtype=np.int64)
            ids = torch.from_numpy(np.resize(motif, n))
        else:
            ids = torch.from_numpy(rng.integers(0, self.vocab, size=n, dtype=np.int64))
        labels = ids.clone()
        if self.prompt_len:
            labels[: self.prompt_len] = -100  # an unsupervised prompt prefix (RL / SFT style records)
        return {"input_ids": ids, "labels": labels}

    def __iter__(self) -> Iterator[List[Dict[str, torch.Tensor]]]:
        if self.interleave_ranks > 1:
            # one process replaying the streams of several data-parallel ranks in turn
            subs = []
            for r in range(self.interleave_ranks):
                d = SyntheticPackedDataset(self.config)
                d.interleave_ranks = 0
                d.dp_rank = r
                subs.append(iter(d))
            while True:
                for it in subs:
                    yield next(it)
        packer = None if self.fill_exact else build_online_packer(self.strategy, self.packing_length, **self.packing_kwargs)
        idx = self.cur_idx
        buf: List[Dict[str, torch.Tensor]] = []
        used = 0
        while self.num_documents is None or idx < int(self.num_documents):
            doc = self._document(idx)
            idx += 1
            n = doc["input_ids"].numel()
            if self.fill_exact:
                room = self.packing_length - used
                if n >= room:
                    buf.append({k: v[:room] for k, v in doc.items()})
                    self.cur_idx = idx
                    yield buf
                    buf, used = [], 0
                else:
                    buf.append(doc)
                    used += n
                continue
            if n > self.packing_length:
                self.cur_idx = idx
                yield [{k: v[: self.packing_length] for k, v in doc.items()}]
                continue
            for pack in packer.add(doc, n):
                # next-fit emits the open pack because THIS document did not fit, so the
                # stream resumes exactly at this document; multi-bucket packers are approximate
                self.cur_idx = idx - 1 if self.strategy == "first_fit" else idx
                yield pack
        if packer is not None:
            for pack in packer.flush():
                self.cur_idx = idx
                yield pack
        elif buf:
            yield buf


class StackCollator:
    """Stacks same-shaped tensors of a list of samples on a new leading dimension."""

    def __call__(self, batch):
        out = {}
        for k in batch[0]:
            vals = [b[k] for b in batch]
            out[k] = torch.stack(vals) if torch.is_tensor(vals[0]) else vals
        return out


@register_dataset("synthetic_tensors")
class SyntheticTensorDataset(IterableDataset):
    """Random tensors by spec, for the image / video / latent trainers:
    ``extra_kwargs.spec = {name: {shape: [...], kind: randn|randint|rand, high: int}}``."""

    def __init__(self, config):
        self.config = config
        self.spec = dict((config.extra_kwargs or {}).get("spec", {}))
        self.seed = int(config.data_seed or 0)
        self.cur_idx = 0
        self.processor = None
        self.dp_rank = 0

    def build(self):
        try:
            from ..parallel import process_group_manager as pgm

            if pgm.process_group_manager is not None:
                self.dp_rank = pgm.process_group_manager.dp_rank
        except Exception:
            pass
        return self

    def get_collator(self):
        return StackCollator()

    def state_dict(self):
        return {"cur_idx": self.cur_idx}

    def load_state_dict(self, sd):
        self.cur_idx = int(sd.get("cur_idx", 0))

    def __iter__(self):
        while True:
            g = torch.Generator().manual_seed(hash((self.seed, self.dp_rank, self.cur_idx)) % (2 ** 31))
            self.cur_idx += 1
            item = {}
            for name, sp in self.spec.items():
                shape = tuple(sp.get("shape", ()))
                kind = sp.get("kind", "randn")
                if kind == "randint":
                    item[name] = torch.randint(0, int(sp.get("high", 2)), shape, generator=g)
                elif kind == "rand":
                    item[name] = torch.rand(shape, generator=g)
                else:
                    item[name] = torch.randn(shape, generator=g)
            yield item


@register_dataset("synthetic_vl")
class SyntheticVisionLanguageDataset(IterableDataset):
    """Packed vision-language samples without files: every sample is ONE document of exactly
    ``packing_length`` tokens in which runs of visual placeholder tokens (one run per image or video)
    alternate with text spans of uniform random ids; pixel values are N(0, 1) in the flattened-patch
    layout the vision towers take, M-RoPE ``(t, h, w)`` positions are precomputed on the host, and the
    loss covers text tokens only.

    ``extra_kwargs``: ``vocab_size``; ``media`` (``"image"`` | ``"video"``); ``num_media`` ``[lo, hi]`` per
    sample; ``size`` ``[lo, hi]`` and ``size_multiple`` (height / width in pixels, multiples of
    ``size_multiple``); ``frames`` ``[lo, hi]`` (videos); ``patch_size``, ``temporal_patch_size``,
    ``merge_size``, ``in_channels``; ``image_token_id``, ``video_token_id``; ``tokens_per_second`` and
    ``second_per_grid`` for the temporal positions of videos; ``pixel_dtype``.
    Samples are a pure function of ``(data_seed, data-parallel rank, index)``; the ranks of one
    sequence-parallel group therefore draw the same sample."""

    def __init__(self, config):
        self.config = config
        kw = dict(config.extra_kwargs or {})
        self.kw = kw
        self.vocab = int(kw.get("vocab_size", 4096))
        self.media = kw.get("media", "image")
        self.num_media = tuple(kw.get("num_media", (1, 2)))
        self.size = tuple(kw.get("size", (56, 112)))
        self.size_multiple = int(kw.get("size_multiple", 28))
        self.frames = tuple(kw.get("frames", (4, 8)))
        self.patch = int(kw.get("patch_size", 14))
        self.tpatch = int(kw.get("temporal_patch_size", 2))
        self.merge = int(kw.get("merge_size", 2))
        self.channels = int(kw.get("in_channels", 3))
        self.image_token_id = int(kw.get("image_token_id", self.vocab - 2))
        self.video_token_id = int(kw.get("video_token_id", self.vocab - 1))
        self.tokens_per_second = float(kw.get("tokens_per_second", 0.0))
        self.second_per_grid = float(kw.get("second_per_grid", 1.0))
        self.pixel_dtype = getattr(torch, kw.get("pixel_dtype", "bfloat16"))
        self.length = int(config.packing_length or 4096)
        self.seed = int(config.data_seed or 0)
        self.dp_rank, self.dp_size = 0, 1
        self.cur_idx = 0
        self.processor = None

    def build(self):
        try:
            from ..parallel import process_group_manager as pgm

            m = pgm.process_group_manager
            if m is not None:
                self.dp_rank, self.dp_size = m.dp_rank, m.dp_size
        except Exception:
            pass
        return self

    def get_collator(self):
        return PackedCollator()

    def state_dict(self) -> Dict[str, Any]:
        return {"cur_idx": self.cur_idx}

    def load_state_dict(self, sd: Dict[str, Any]) -> None:
        self.cur_idx = int(sd.get("cur_idx", 0))

    def sample(self, idx: int) -> Dict[str, torch.Tensor]:
        from ..models.mrope import mrope_positions_one

        rng = np.random.default_rng([self.seed, self.dp_rank, idx])
        video = self.media == "video"
        n_media = int(rng.integers(self.num_media[0], self.num_media[1] + 1))
        grids, counts = [], []
        for _ in range(n_media):
            h, w = (int(rng.integers(self.size[0] // self.size_multiple, self.size[1] // self.size_multiple + 1)) * self.size_multiple
                    for _ in range(2))
            t = int(rng.integers(self.frames[0], self.frames[1] + 1)) // self.tpatch if video else 1
            g = (max(t, 1), h // self.patch, w // self.patch)
            cnt = g[0] * (g[1] // self.merge) * (g[2] // self.merge)
            if sum(counts) + cnt + 2 * (len(counts) + 2) > self.length:
                break  # the next medium would not leave room for any text
            grids.append(g)
            counts.append(cnt)
        n_text = self.length - sum(counts)
        # text spans: one before every medium and one at the end, at least one token each
        cuts = np.sort(rng.choice(np.arange(1, n_text), size=len(grids), replace=False)) if grids else np.array([], dtype=np.int64)
        spans = np.diff(np.concatenate([[0], cuts, [n_text]])).astype(np.int64)
        tok = self.video_token_id if video else self.image_token_id
        text_vocab = min(self.vocab, self.image_token_id, self.video_token_id)
        parts, labels = [], []
        for i, span in enumerate(spans):
            t_ids = rng.integers(0, text_vocab, size=int(span), dtype=np.int64)
            parts.append(t_ids)
            labels.append(t_ids.copy())
            if i < len(grids):
                parts.append(np.full(counts[i], tok, dtype=np.int64))
                labels.append(np.full(counts[i], -100, dtype=np.int64))
        ids = np.concatenate(parts)
        pos, used = mrope_positions_one(ids, (self.image_token_id, self.video_token_id), grids,
                                        [self.second_per_grid] * len(grids) if video else None, self.merge,
                                        self.tokens_per_second if video else 0.0)
        assert used == len(grids) and ids.shape[0] == self.length
        n_patches = sum(g[0] * g[1] * g[2] for g in grids)
        feat = self.channels * self.tpatch * self.patch * self.patch
        gen = torch.Generator().manual_seed(int(rng.integers(0, 2 ** 31 - 1)))
        pixels = torch.randn(n_patches, feat, generator=gen).to(self.pixel_dtype)
        out = {"input_ids": torch.from_numpy(ids), "labels": torch.from_numpy(np.concatenate(labels)),
               "position_ids": torch.from_numpy(pos)}
        grid_t = torch.tensor(grids, dtype=torch.long).view(-1, 3)
        if video:
            out["pixel_values_videos"], out["video_grid_thw"] = pixels, grid_t
        else:
            out["pixel_values"], out["image_grid_thw"] = pixels, grid_t
        return out

    def __iter__(self):
        while True:
            idx = self.cur_idx
            self.cur_idx += 1
            yield [self.sample(idx)]
