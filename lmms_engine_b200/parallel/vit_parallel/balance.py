"""Deterministic, locality-aware longest-processing-time planner for vision frames: ranks hold
different numbers of patches per step; frames are re-assigned so that every rank runs the ViT on
a near-equal patch count, preferring to keep a frame on the rank that already holds it.  The
assignment runs in the C++ host library (``csrc/host/packing.cpp``).  Reference:
src/lmms_engine/parallel/vit_parallel/balance.py:22-195."""
from __future__ import annotations

import ctypes
from typing import List, Sequence, Tuple

from ... import _native


def lpt_balance(weights: Sequence[int], home: Sequence[int], ranks: int, slack: float = 0.25) -> Tuple[List[int], List[int]]:
    """Owner rank of every item and the resulting per-rank load.  Identical on every rank."""
    n = len(weights)
    lib = _native.lib("packing")
    fn = lib.lpt_balance
    fn.restype = None
    fn.argtypes = [ctypes.POINTER(ctypes.c_long), ctypes.POINTER(ctypes.c_int), ctypes.c_long, ctypes.c_int, ctypes.c_double,
                   ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_long)]
    w = (ctypes.c_long * max(n, 1))(*[int(x) for x in weights])
    h = (ctypes.c_int * max(n, 1))(*[int(x) for x in home])
    owner = (ctypes.c_int * max(n, 1))()
    load = (ctypes.c_long * ranks)()
    fn(w, h, n, ranks, float(slack), owner, load)
    return [owner[i] for i in range(n)], [load[r] for r in range(ranks)]


def plan_frame_exchange(frames_per_rank: List[List[int]], slack: float = 0.25):
    """``frames_per_rank[r]`` = patch counts of the frames rank r holds.  Returns
    ``owner[r][i]`` (destination of rank r's i-th frame) and, per rank, the send / receive patch
    counts ``send[r][dst]`` for the all-to-all."""
    ranks = len(frames_per_rank)
    flat_w, flat_home = [], []
    for r, fr in enumerate(frames_per_rank):
        flat_w += list(fr)
        flat_home += [r] * len(fr)
    owner_flat, load = lpt_balance(flat_w, flat_home, ranks, slack)
    owner, send, k = [], [[0] * ranks for _ in range(ranks)], 0
    for r, fr in enumerate(frames_per_rank):
        owner.append(owner_flat[k:k + len(fr)])
        for w, o in zip(fr, owner[-1]):
            send[r][o] += w
        k += len(fr)
    return owner, send, load
