"""Collator that emits the packed form the native models consume directly: a flat token
stream with ``cu_seqlens`` and per-document positions (no padded ``[n_docs, L]`` detour).
Multimodal tensors are concatenated on dim 0 as in the reference collator
(src/lmms_engine/datasets/collator/vision_collator.py:24-65)."""
from __future__ import annotations

from typing import Any, Dict, List, Sequence

import torch


def _flatten(batch: Sequence[Any]) -> List[Dict[str, Any]]:
    out: List[Dict[str, Any]] = []
    for item in batch:
        if isinstance(item, (list, tuple)):
            out.extend(item)
        else:
            out.append(item)
    return out


class PackedCollator:
    def __init__(self, pad_to_multiple_of: int = 1, ignore_index: int = -100):
        self.multiple = int(pad_to_multiple_of)
        self.ignore_index = ignore_index

    def __call__(self, batch: Sequence[Any]) -> Dict[str, torch.Tensor]:
        samples = _flatten(batch)
        ids = [s["input_ids"].view(-1) for s in samples]
        labels = [s.get("labels", s["input_ids"]).view(-1) for s in samples]
        lens = torch.tensor([t.numel() for t in ids], dtype=torch.int32)
        cu = torch.zeros(len(ids) + 1, dtype=torch.int32)
        cu[1:] = torch.cumsum(lens, 0)
        out: Dict[str, torch.Tensor] = {
            "input_ids": torch.cat(ids),
            "labels": torch.cat(labels),
            "cu_seqlens": cu,
            "position_ids": torch.cat([torch.arange(n, dtype=torch.long) for n in lens.tolist()]),
        }
        if any("position_ids" in s for s in samples):  # multimodal (3, n) positions from a processor
            out["position_ids"] = torch.cat([s["position_ids"] for s in samples], dim=-1)
        keys = list(dict.fromkeys(k for s in samples for k in s.keys()))  # a text-only first sample must not hide the others' media
        for key in keys:
            if key in ("input_ids", "labels", "position_ids", "attention_mask"):
                continue
            vals = [s[key] for s in samples if key in s and s[key] is not None]
            if vals and all(torch.is_tensor(v) for v in vals):
                out[key] = torch.cat(vals, dim=0)
        return out
