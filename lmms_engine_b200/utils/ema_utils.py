"""Exponential moving average of the weights on flat or per-parameter fp32 shadows.

Same options as the reference helper (src/lmms_engine/utils/ema_utils.py:11-147):
``decay``, ``update_every``, ``start_step``, ``requires_grad_only``, a name filter with
``mode: substring|regex`` and ``include`` / ``exclude`` lists, and resuming training from
the EMA weights.  DTensor parameters are averaged shard-locally.
"""
from __future__ import annotations

import re
from typing import Any, Dict, Iterable, Optional

import torch

from ..ops import optim as optim_ops


def _local(t: torch.Tensor) -> torch.Tensor:
    return t._local_tensor if hasattr(t, "_local_tensor") else t


class EMAHelper:
    def __init__(self, model: torch.nn.Module, decay: float = 0.9999, update_every: int = 1, start_step: int = 0,
                 requires_grad_only: bool = True, param_filter: Optional[Dict[str, Any]] = None, enabled: bool = True):
        self.model = model
        self.decay = decay
        self.update_every = max(int(update_every), 1)
        self.start_step = int(start_step)
        self.requires_grad_only = requires_grad_only
        self.param_filter = param_filter or {}
        self.enabled = enabled
        self.shadow: Dict[str, torch.Tensor] = {}
        self.initialized = False

    def _selected(self, name: str, p: torch.nn.Parameter) -> bool:
        if self.requires_grad_only and not p.requires_grad:
            return False
        mode = self.param_filter.get("mode", "substring")
        inc, exc = self.param_filter.get("include"), self.param_filter.get("exclude")

        def hit(pats: Iterable[str]) -> bool:
            if mode == "regex":
                return any(re.search(pt, name) for pt in pats)
            return any(pt in name for pt in pats)

        if inc and not hit(inc):
            return False
        if exc and hit(exc):
            return False
        return True

    def maybe_init(self) -> None:
        if not self.enabled or self.initialized:
            return
        for name, p in self.model.named_parameters():
            if self._selected(name, p):
                self.shadow[name] = _local(p.detach()).float().clone()
        self.initialized = True

    @torch.no_grad()
    def update(self, step: int) -> None:
        if not self.enabled or step < self.start_step or step % self.update_every != 0:
            return
        self.maybe_init()
        for name, p in self.model.named_parameters():
            sh = self.shadow.get(name)
            if sh is None:
                continue
            src = _local(p.detach())
            if src.is_cuda and src.dtype in (torch.bfloat16, torch.float32) and src.is_contiguous():
                optim_ops.ema_update(sh.view(-1), src.view(-1), self.decay)
            else:
                sh.mul_(self.decay).add_(src.float(), alpha=1.0 - self.decay)

    def state_dict(self) -> Dict[str, torch.Tensor]:
        return {k: v.detach().cpu() for k, v in self.shadow.items()}

    def load_state_dict(self, sd: Dict[str, torch.Tensor]) -> None:
        self.maybe_init()
        for k, v in sd.items():
            if k in self.shadow:
                self.shadow[k].copy_(_local(v))

    @torch.no_grad()
    def copy_to_model(self) -> None:
        """Overwrite the live weights with the averaged ones (``ema_resume_from_ema``)."""
        for name, p in self.model.named_parameters():
            if name in self.shadow:
                _local(p.data).copy_(self.shadow[name])
