"""Masking collator for diffusion LMs: every sequence draws ``t ~ U[p_min, p_max]`` and masks
each token with probability ``t``; returns the packed stream plus ``mlm_prob`` per token
(reference: src/lmms_engine/datasets/collator/text_dllm_collator.py:1-126)."""
from __future__ import annotations

from typing import Any, Dict, Sequence

import torch

from .packed_collator import PackedCollator, _flatten


class TextDllmCollator:
    def __init__(self, mask_token_id: int, p_min: float = 0.05, p_max: float = 1.0, seed: int = 0):
        self.mask_token_id, self.p_min, self.p_max = mask_token_id, p_min, p_max
        self.gen = torch.Generator().manual_seed(seed)
        self.base = PackedCollator()

    def __call__(self, batch: Sequence[Any]) -> Dict[str, torch.Tensor]:
        out = self.base(batch)
        ids = out["input_ids"]
        cu = out["cu_seqlens"].tolist()
        t_tok = torch.empty(ids.numel())
        for a, b in zip(cu[:-1], cu[1:]):
            t = self.p_min + (self.p_max - self.p_min) * torch.rand((), generator=self.gen)
            t_tok[a:b] = t
        mask = torch.rand(ids.numel(), generator=self.gen) < t_tok
        if "labels" in out:
            mask &= out["labels"] != -100  # only supervised tokens can be masked
        out["labels"] = torch.where(mask, ids, torch.full_like(ids, -100))
        out["input_ids"] = torch.where(mask, torch.full_like(ids, self.mask_token_id), ids)
        out["mlm_prob"] = t_tok
        return out
