"""Offline packing of map-style datasets into index groups
(reference: src/lmms_engine/datasets/naive/multimodal_dataset.py:205-237)."""
from __future__ import annotations

import ctypes
from typing import List, Sequence

from ... import _native


def _run(fn_name: str, lengths: Sequence[int], capacity: int, *extra) -> List[List[int]]:
    lib = _native.lib("packing")
    n = len(lengths)
    arr = (ctypes.c_long * n)(*[int(x) for x in lengths])
    out = (ctypes.c_long * n)()
    fn = getattr(lib, fn_name)
    fn.restype = ctypes.c_long
    fn.argtypes = [ctypes.POINTER(ctypes.c_long), ctypes.c_long, ctypes.c_long] + [ctypes.c_long] * len(extra) + [ctypes.POINTER(ctypes.c_long)]
    groups = fn(arr, n, int(capacity), *[int(e) for e in extra], out)
    res: List[List[int]] = [[] for _ in range(groups)]
    for i in range(n):
        res[out[i]].append(i)
    return res


def pack_by_first_fit(lengths: Sequence[int], packing_length: int) -> List[List[int]]:
    return _run("offline_first_fit", lengths, packing_length)


def pack_by_window(lengths: Sequence[int], packing_length: int, window: int) -> List[List[int]]:
    return _run("offline_window", lengths, packing_length, window)


def build_offline_groups(strategy: str, lengths: Sequence[int], packing_length: int) -> List[List[int]]:
    if strategy in (None, "first_fit"):
        return pack_by_first_fit(lengths, packing_length)
    if strategy.startswith("window_"):
        return pack_by_window(lengths, packing_length, int(strategy.split("_", 1)[1]))
    raise ValueError(f"unknown offline packing strategy '{strategy}'")
