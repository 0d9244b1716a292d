"""Learning-rate schedules: ``cosine`` (``min_lr_ratio``, ``num_cycles``), ``wsd``
(warm-up / stable / decay with ``stable_ratio`` and ``min_lr_ratio``) and ``constant``
(linear warm-up from ``start_factor``).  Same shapes as the reference
(src/lmms_engine/utils/fsdp2_utils.py:119-232)."""
from __future__ import annotations

import math

from torch.optim.lr_scheduler import LambdaLR


def cosine_lambda(step, warmup, total, min_lr_ratio=0.0, num_cycles=0.5):
    if step < warmup:
        return float(step) / float(max(1, warmup))
    prog = float(step - warmup) / float(max(1, total - warmup))
    prog = min(prog, 1.0)
    c = 0.5 * (1.0 + math.cos(math.pi * float(num_cycles) * 2.0 * prog))
    return min_lr_ratio + (1.0 - min_lr_ratio) * max(0.0, c)


def wsd_lambda(step, warmup, total, stable_ratio=0.9, min_lr_ratio=0.0):
    if step < warmup:
        return float(step) / float(max(1, warmup))
    stable_end = warmup + int((total - warmup) * stable_ratio)
    if step < stable_end:
        return 1.0
    prog = float(step - stable_end) / float(max(1, total - stable_end))
    prog = min(prog, 1.0)
    return min_lr_ratio + (1.0 - min_lr_ratio) * 0.5 * (1.0 + math.cos(math.pi * prog))


def constant_lambda(step, warmup, start_factor=0.01):
    if warmup <= 0 or step >= warmup:
        return 1.0
    return start_factor + (1.0 - start_factor) * float(step) / float(warmup)


def lr_factor(name: str, step: int, warmup: int, total: int, **kw) -> float:
    if name == "cosine":
        return cosine_lambda(step, warmup, total, kw.get("min_lr_ratio", 0.0), kw.get("num_cycles", 0.5))
    if name == "wsd":
        return wsd_lambda(step, warmup, total, kw.get("stable_ratio", 0.9), kw.get("min_lr_ratio", 0.0))
    if name in ("constant", "constant_with_warmup"):
        return constant_lambda(step, warmup, kw.get("start_factor", 0.01))
    if name == "linear":
        if step < warmup:
            return float(step) / float(max(1, warmup))
        return max(0.0, float(total - step) / float(max(1, total - warmup)))
    raise ValueError(f"unknown lr_scheduler_type '{name}'")


def build_scheduler(optimizer, name: str, warmup: int, total: int, **kw) -> LambdaLR:
    return LambdaLR(optimizer, lambda s: lr_factor(name, s, warmup, total, **kw))
