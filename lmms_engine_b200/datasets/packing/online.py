"""Online packers: thin item-keeping shells over the native ``PackStream`` core."""
from __future__ import annotations

import ctypes
from typing import Any, Dict, Iterator, List

from ... import _native
from .base import OnlinePackingStrategy

_lib = None


def _core():
    global _lib
    if _lib is None:
        lib = _native.lib("packing")
        lib.pack_stream_new.restype = ctypes.c_void_p
        lib.pack_stream_new.argtypes = [ctypes.c_int, ctypes.c_long, ctypes.c_int, ctypes.c_double, ctypes.c_int, ctypes.c_long]
        lib.pack_stream_free.argtypes = [ctypes.c_void_p]
        lib.pack_stream_add.argtypes = [ctypes.c_void_p, ctypes.c_long, ctypes.c_long]
        lib.pack_stream_flush.argtypes = [ctypes.c_void_p]
        lib.pack_stream_ready.argtypes = [ctypes.c_void_p]
        lib.pack_stream_ready.restype = ctypes.c_int
        lib.pack_stream_pop.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_long), ctypes.c_long]
        lib.pack_stream_pop.restype = ctypes.c_long
        _lib = lib
    return _lib


class _NativeStreamPacker(OnlinePackingStrategy):
    policy = 0

    def __init__(self, packing_length: int, max_open: int = 1, fill_threshold: float = 1.0, max_swap_iters: int = 200,
                 min_gain: int = 1) -> None:
        super().__init__(packing_length)
        self._args = (self.policy, int(packing_length), int(max_open), float(fill_threshold), int(max_swap_iters), int(min_gain))
        self._h = _core().pack_stream_new(*self._args)
        self._items: Dict[int, Any] = {}
        self._next = 0
        self._buf = (ctypes.c_long * 4096)()

    def __del__(self):
        try:
            if getattr(self, "_h", None):
                _core().pack_stream_free(self._h)
                self._h = None
        except Exception:
            pass

    def _drain(self) -> Iterator[List[Any]]:
        lib = _core()
        while lib.pack_stream_ready(self._h) > 0:
            n = lib.pack_stream_pop(self._h, self._buf, len(self._buf))
            if n < -1:
                self._buf = (ctypes.c_long * (-n))()
                continue
            if n < 0:
                break
            yield [self._items.pop(self._buf[i]) for i in range(n)]

    def add(self, item: Any, length: int) -> Iterator[List[Any]]:
        if length > self.packing_length:
            raise ValueError(f"sample of length {length} exceeds packing_length {self.packing_length}")
        i = self._next
        self._next += 1
        self._items[i] = item
        _core().pack_stream_add(self._h, i, int(length))
        yield from self._drain()

    def flush(self) -> Iterator[List[Any]]:
        _core().pack_stream_flush(self._h)
        yield from self._drain()


class FirstFitPacking(_NativeStreamPacker):
    """One open pack; it is emitted when the next sample does not fit (next-fit, the
    behaviour the reference ships under the name ``first_fit``)."""

    policy = 0

    def __init__(self, packing_length: int) -> None:
        super().__init__(packing_length, 1, 1.0)


class BestFitPacking(_NativeStreamPacker):
    policy = 1

    def __init__(self, packing_length: int, num_open_buckets: int = 4, fill_threshold: float = 0.95) -> None:
        if num_open_buckets < 1:
            raise ValueError("num_open_buckets must be >= 1")
        if not 0.0 < fill_threshold <= 1.0:
            raise ValueError("fill_threshold must be in (0, 1]")
        super().__init__(packing_length, num_open_buckets, fill_threshold)


class BalancedPacking(_NativeStreamPacker):
    policy = 2

    def __init__(self, packing_length: int, num_buckets: int = 8, max_swap_iters: int = 200, min_gain: int = 1) -> None:
        if num_buckets < 1:
            raise ValueError("num_buckets must be >= 1")
        super().__init__(packing_length, num_buckets, 1.0, max_swap_iters, min_gain)


class TrueFirstFitPacking(_NativeStreamPacker):
    """First-fit over several open packs (earlier packs are revisited)."""

    policy = 3

    def __init__(self, packing_length: int, num_open_buckets: int = 8, fill_threshold: float = 0.98) -> None:
        super().__init__(packing_length, num_open_buckets, fill_threshold)


ONLINE_PACKERS = {
    "first_fit": FirstFitPacking,
    "best_fit": BestFitPacking,
    "balanced": BalancedPacking,
    "true_first_fit": TrueFirstFitPacking,
}


def build_online_packer(name: str, packing_length: int, **kwargs) -> OnlinePackingStrategy:
    if name not in ONLINE_PACKERS:
        raise ValueError(f"unknown online packing strategy '{name}', expected one of {sorted(ONLINE_PACKERS)}")
    return ONLINE_PACKERS[name](packing_length, **kwargs)
