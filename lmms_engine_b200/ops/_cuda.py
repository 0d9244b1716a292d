"""ctypes glue between torch tensors and the native launchers.

Each exported function is declared once with a compact signature string:
``p`` device/host pointer, ``i`` int32, ``l`` int64, ``f`` float, ``s`` CUDA stream.
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, Optional, Tuple

import torch

from .. import _native

_SIG: Dict[str, Tuple[str, str]] = {
    # gemm_sm100
    "b200_gemm_bf16": ("gemm_sm100", "pppiiiiiiiiffppiiips"),
    "b200_gemm_swiglu_bf16": ("gemm_sm100", "ppppppiiiiiiips"),
    "b200_gemm_stats_bf16": ("gemm_sm100", "ppppiiiiiifps"),
    "b200_gemm_tile_n": ("gemm_sm100", ""),
    "b200_gemm_set_pair_mode": ("gemm_sm100", "i"),
    "b200_gemm_pair_clusters": ("gemm_sm100", ""),
    # elementwise
    "b200_num_partials": ("elementwise", ""),
    "b200_norm_fwd": ("elementwise", "ppppppppiiffis"),
    "b200_norm_bwd": ("elementwise", "pppppppppppiifiis"),
    "b200_rope_table": ("elementwise", "ppppiiiiiifs"),
    "b200_rope_apply": ("elementwise", "ppppiiiillis"),
    "b200_swiglu_fwd": ("elementwise", "pppls"),
    "b200_swiglu_bwd": ("elementwise", "pppppls"),
    "b200_adamw": ("elementwise", "pppppilfffffffpps"),
    "b200_muon_momentum": ("elementwise", "ppipplfipfs"),
    "b200_muon_update": ("elementwise", "ppplfffps"),
    "b200_ema": ("elementwise", "ppilfs"),
    "b200_sumsq": ("elementwise", "pilppis"),
    "b200_clip_coef": ("elementwise", "ppppfps"),
    "b200_scale": ("elementwise", "pilps"),
    "b200_gather_rows": ("elementwise", "pppli" + "lps"),
    "b200_scatter_rows": ("elementwise", "ppplis" + ""),
    "b200_ce_finalize": ("elementwise", "pppppiiliis"),
    "b200_ce_dlogits": ("elementwise", "ppppiliis"),
}
_SIG["b200_scatter_rows"] = ("elementwise", "pppliilps")

_CT = {"p": ctypes.c_void_p, "i": ctypes.c_int, "l": ctypes.c_long, "f": ctypes.c_float, "s": ctypes.c_void_p}
_fn_cache: Dict[str, ctypes._CFuncPtr] = {}
_status: Dict[int, torch.Tensor] = {}
launch_count = 0  # number of native kernel-launching calls made by this process


def register(name: str, libname: str, sig: str) -> None:
    _SIG[name] = (libname, sig)


def fn(name: str):
    f = _fn_cache.get(name)
    if f is None:
        libname, sig = _SIG[name]
        f = getattr(_native.lib(libname), name)
        f.argtypes = [_CT[c] for c in sig]
        f.restype = ctypes.c_int
        _fn_cache[name] = f
    return f


def ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def status_word(device: torch.device) -> torch.Tensor:
    """Per-device int32 word that kernels raise on a bounded-wait timeout."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    t = _status.get(idx)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
        _status[idx] = t
    return t


STATUS_NAMES = {1: "a barrier wait timed out", 2: "bad shape", 3: "a wait for a peer GPU timed out", 4: "a receive buffer overflowed",
                5: "an index table addressed a row outside its tensor (the access was skipped)"}


def check_status(device: Optional[torch.device] = None) -> None:
    """Synchronising check of the kernel status word; raises on a device-side timeout."""
    for idx, t in list(_status.items()):
        if device is not None and device.index not in (None, idx):
            continue
        v = int(t.item())
        if v != 0:
            t.zero_()
            raise RuntimeError(f"native kernel reported status {v} on cuda:{idx} ({STATUS_NAMES.get(v, 'unknown')})")
    if _native.DEBUG_BOUNDS and "b200_moe_debug_bad_index" in _SIG and fn("b200_moe_debug_bad_index")() > 0:
        raise RuntimeError("debug build: the expert permutation computed a row outside its tables (counts and top-k indices disagree)")


# LMMS_B200_DEBUG_SYNC=1: synchronise after every native launch and name the launcher whose kernel failed
# (asynchronous faults are otherwise reported by whatever call happens to synchronise next).
DEBUG_SYNC = os.environ.get("LMMS_B200_DEBUG_SYNC", "0") == "1"


def _debug_sync(name: str) -> None:
    try:
        torch.cuda.synchronize()
    except Exception as e:  # noqa: BLE001
        raise RuntimeError(f"device fault during or before {name}: {e}") from e


def call(name: str, *args) -> None:
    global launch_count
    rc = fn(name)(*args)
    launch_count += 1
    if rc != 0:
        raise RuntimeError(f"{name} failed with code {rc}")
    if DEBUG_SYNC:
        _debug_sync(name)


def call_raw(name: str, *args) -> int:
    """Like ``call`` for launchers whose return value carries information (negative = error)."""
    global launch_count
    rc = fn(name)(*args)
    launch_count += 1
    if DEBUG_SYNC:
        _debug_sync(name)
    return rc


def require_bf16_cuda(*ts: torch.Tensor) -> None:
    for t in ts:
        if t is None:
            continue
        if not t.is_cuda or t.dtype != torch.bfloat16:
            raise TypeError(f"native path needs CUDA bf16 tensors, got {t.device} {t.dtype}")
