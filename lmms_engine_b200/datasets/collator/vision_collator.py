"""Padded-batch collator with the reference's batch contract
(src/lmms_engine/datasets/collator/vision_collator.py:12-69): packs are flattened, ``input_ids``
padded with the pad id and ``labels`` with -100 (right or left), ``attention_mask =
input_ids != pad``, every other tensor concatenated on dim 0."""
from __future__ import annotations

from typing import Any, Dict, Sequence

import torch

from .packed_collator import _flatten


class VisionCollator:
    STACKED = ("video",)

    def __init__(self, processor=None, pad_token_id: int = 0, padding_side: str = "right", ignore_index: int = -100):
        self.processor = processor
        tok = getattr(processor, "tokenizer", None)
        if tok is not None and getattr(tok, "pad_token_id", None) is not None:
            pad_token_id = tok.pad_token_id
            padding_side = getattr(tok, "padding_side", padding_side)
        self.pad, self.side, self.ignore = pad_token_id, padding_side, ignore_index

    def _pad(self, seqs, value):
        L = max(s.numel() for s in seqs)
        out = seqs[0].new_full((len(seqs), L), value)
        for i, s in enumerate(seqs):
            if self.side == "left":
                out[i, L - s.numel() :] = s
            else:
                out[i, : s.numel()] = s
        return out

    def __call__(self, batch: Sequence[Any]) -> Dict[str, torch.Tensor]:
        samples = _flatten(batch)
        ids = self._pad([s["input_ids"].view(-1) for s in samples], self.pad)
        out: Dict[str, torch.Tensor] = {"input_ids": ids}
        if all("labels" in s for s in samples):  # generative families carry prompts without labels
            out["labels"] = self._pad([s["labels"].view(-1) for s in samples], self.ignore)
        lens = torch.tensor([s["input_ids"].numel() for s in samples])
        ar = torch.arange(ids.shape[1]).unsqueeze(0)
        if self.side == "left":
            out["attention_mask"] = (ar >= (ids.shape[1] - lens).unsqueeze(1)).long()
        else:
            out["attention_mask"] = (ar < lens.unsqueeze(1)).long()
        for key in samples[0].keys():
            if key in ("input_ids", "labels", "attention_mask"):
                continue
            vals = [s[key] for s in samples if key in s and s[key] is not None]
            if vals and all(torch.is_tensor(v) for v in vals):
                # a clip is one item of the batch (its first axis is time), everything else is a list of rows
                out[key] = torch.stack(vals, 0) if key in self.STACKED else self.join(key, vals)
            elif vals and isinstance(vals[0], (bool, int, float)):
                out[key] = vals[0]  # a flag of the whole batch (``use_audio_in_video``)
        return out

    def join(self, key: str, vals):
        return torch.cat(vals, dim=0)


class LLaVACollator(VisionCollator):
    """The padded collator for processors that give every image as ``[1, tiles, C, H, W]`` with its own number of tiles
    (src/lmms_engine/datasets/collator/llava_collator.py:14-89): ``pixel_values`` are zero-padded on the tile axis to the
    largest count of the batch before they are concatenated; rows that already agree pass unchanged."""

    def join(self, key: str, vals):
        if key == "pixel_values" and vals[0].dim() >= 3 and len({v.shape[1] for v in vals}) > 1:
            most = max(v.shape[1] for v in vals)
            vals = [torch.cat([v, v.new_zeros((v.shape[0], most - v.shape[1]) + tuple(v.shape[2:]))], 1) if v.shape[1] < most else v
                    for v in vals]
        return torch.cat(vals, dim=0)
