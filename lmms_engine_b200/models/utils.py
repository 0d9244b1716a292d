"""Model FLOPs accounting used for MFU.

Same formulas as the reference counter (src/lmms_engine/models/utils.py:48-292):
``6 * N_dense * tokens + 12 * sum(seqlen^2) * head_dim * heads * layers`` for dense
Qwen-style decoders, the activated-parameter variant for MoE; vision-tower FLOPs are not
counted (docs/reference/mfu.md:160-166).
"""
from __future__ import annotations

from typing import Any, Iterable, Optional, Sequence

import torch


def _get(cfg: Any, name: str, default=None):
    if isinstance(cfg, dict):
        return cfg.get(name, default)
    return getattr(cfg, name, default)


class FlopsCounter:
    """``estimate_flops(batch_seqlens, delta_time) -> (achieved TFLOP/s, promised TFLOP/s)``."""

    def __init__(self, config: Any):
        text_cfg = _get(config, "text_config", None) or config
        self.config = text_cfg
        self.model_type = _get(config, "model_type", "qwen2")

    # -- parameter counts -------------------------------------------------------------
    def dense_params(self) -> int:
        c = self.config
        H, L, V = _get(c, "hidden_size"), _get(c, "num_hidden_layers"), _get(c, "vocab_size")
        nq, nkv = _get(c, "num_attention_heads"), _get(c, "num_key_value_heads")
        D = _get(c, "head_dim", None) or H // nq
        I = _get(c, "intermediate_size")
        attn = H * (nq * D + 2 * nkv * D) + nq * D * H
        n_exp = _get(c, "num_experts", 0) or 0
        if n_exp:
            Ie = _get(c, "moe_intermediate_size")
            topk = _get(c, "num_experts_per_tok")
            mlp = 3 * H * Ie * topk + H * n_exp
            shared = _get(c, "shared_expert_intermediate_size", 0) or 0
            mlp += 3 * H * shared
        else:
            mlp = 3 * H * I
        return L * (attn + mlp) + 2 * V * H

    def flops_per_step(self, seqlens: Sequence[int]) -> float:
        c = self.config
        H, L = _get(c, "hidden_size"), _get(c, "num_hidden_layers")
        nq = _get(c, "num_attention_heads")
        D = _get(c, "head_dim", None) or H // nq
        tokens = float(sum(seqlens))
        sq = float(sum(int(s) * int(s) for s in seqlens))
        return 6.0 * self.dense_params() * tokens + 12.0 * sq * D * nq * L

    def estimate_flops(self, batch_seqlens: Sequence[int], delta_time: float):
        from ..utils.train_utils import TrainUtilities

        achieved = self.flops_per_step(batch_seqlens) / max(delta_time, 1e-9) / 1e12
        return achieved, TrainUtilities.get_device_flops("T")


def setup_flops_counter(config: Any) -> FlopsCounter:
    return FlopsCounter(config)
