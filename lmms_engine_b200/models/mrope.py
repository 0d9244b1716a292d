"""Multimodal rotary position ids ``[3, T]`` (temporal, height, width) for packed streams.

Text tokens advance all three streams together.  A run of vision placeholder tokens that
stands for a ``(t, h, w)`` patch grid (``h/m x w/m`` merged tokens per temporal step) gets the
temporal index ``floor(frame * seconds_per_grid * tokens_per_second)`` (0 for images and for
Qwen3-VL, whose frames are separated by timestamp text), the row index and the column index
of each merged token, all offset by the running position; text after the run resumes at
``max(position) + 1``.  Every document of a packed stream restarts at 0.  Host-side numpy;
behaviour of ``qwen2_5_vl_rope_index`` / ``qwen3_vl_get_rope_index`` in the reference
(src/lmms_engine/models/common_ops/rope.py:8-346).
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch


def _runs(mask: np.ndarray) -> List[Tuple[int, int]]:
    if not mask.any():
        return []
    d = np.diff(np.concatenate([[0], mask.astype(np.int8), [0]]))
    return list(zip(np.nonzero(d == 1)[0].tolist(), np.nonzero(d == -1)[0].tolist()))


def mrope_positions_one(ids: np.ndarray, vision_ids: Sequence[int], grids: List[Tuple[int, int, int]],
                        seconds: Optional[List[float]], merge: int, tokens_per_second: float) -> Tuple[np.ndarray, int]:
    """Positions ``[3, n]`` of one document and the number of grids consumed."""
    n = ids.shape[0]
    pos = np.zeros((3, n), dtype=np.int64)
    is_vis = np.isin(ids, np.asarray(list(vision_ids)))
    cur = 0  # next position value
    at = 0  # cursor in the stream
    used = 0
    for lo, hi in _runs(is_vis):
        # text before the run
        if lo > at:
            pos[:, at:lo] = np.arange(lo - at)[None] + cur
            cur += lo - at
        p = lo
        while p < hi:
            if used >= len(grids):
                raise ValueError("more vision placeholder runs than grids")
            t, h, w = grids[used]
            gh, gw = h // merge, w // merge
            cnt = t * gh * gw
            if p + cnt > hi:
                raise ValueError(f"placeholder run of {hi - p} tokens does not match grid {grids[used]} ({cnt} tokens)")
            sec = seconds[used] if seconds is not None else 0.0
            ti = np.floor(np.arange(t) * sec * tokens_per_second).astype(np.int64)
            pos[0, p:p + cnt] = np.repeat(ti, gh * gw) + cur
            pos[1, p:p + cnt] = np.tile(np.repeat(np.arange(gh), gw), t) + cur
            pos[2, p:p + cnt] = np.tile(np.arange(gw), t * gh) + cur
            cur = int(pos[:, p:p + cnt].max()) + 1
            p += cnt
            used += 1
        at = hi
    if at < n:
        pos[:, at:] = np.arange(n - at)[None] + cur
    return pos, used


def build_mrope_positions(input_ids, cu_seqlens, vision_token_ids: Sequence[int], grids, seconds=None, merge: int = 2,
                          tokens_per_second: float = 0.0) -> torch.Tensor:
    """Positions for a packed stream: ``input_ids [T]``, ``cu_seqlens [n+1]``; ``grids`` lists the
    ``(t, h, w)`` of every image / video in order of appearance over the whole stream."""
    ids = input_ids.cpu().numpy() if torch.is_tensor(input_ids) else np.asarray(input_ids)
    cu = cu_seqlens.cpu().tolist() if torch.is_tensor(cu_seqlens) else list(cu_seqlens)
    grids = [(int(a), int(b), int(c)) for a, b, c in (grids.tolist() if torch.is_tensor(grids) else grids)]
    seconds = list(seconds.tolist() if torch.is_tensor(seconds) else seconds) if seconds is not None else None
    out = np.zeros((3, ids.shape[0]), dtype=np.int64)
    g = 0
    for d in range(len(cu) - 1):
        lo, hi = cu[d], cu[d + 1]
        pos, used = mrope_positions_one(ids[lo:hi], vision_token_ids, grids[g:], seconds[g:] if seconds is not None else None,
                                        merge, tokens_per_second)
        out[:, lo:hi] = pos
        g += used
    return torch.from_numpy(out)
