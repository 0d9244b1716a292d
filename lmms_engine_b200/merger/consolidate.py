"""Turn per-rank DTensor shards back into full tensors.

Works from what each saved DTensor records about itself - placements, mesh shape and the
local shard - without needing a process group: for a 1-D mesh shards are concatenated on
``Shard.dim`` (or one replica is taken); for multi-axis meshes (FSDP x EP, HSDP) the mesh
axes are folded from the innermost outwards.  ``Shard`` on a mesh axis of size 1 and the
zero-size tail shards that uneven chunking produces are handled.  Behavioural counterpart:
``FSDP2Merger.consolidate`` (src/lmms_engine/merger/fsdp2.py:86-276).
"""
from __future__ import annotations

from typing import Any, Dict, List, Sequence, Tuple

import torch


def _describe(t: Any):
    """(local tensor, placements as [('S', dim) | ('R',)], mesh shape) of one saved value."""
    if hasattr(t, "placements") and hasattr(t, "_local_tensor"):
        pl = []
        for p in t.placements:
            if getattr(p, "is_shard", lambda: False)():
                pl.append(("S", int(p.dim)))
            else:
                pl.append(("R",))
        return t._local_tensor, pl, tuple(t.device_mesh.shape)
    return t, None, None


def fold_axis(pieces: Sequence[torch.Tensor], placement: Tuple, full_dim_size: int = -1) -> torch.Tensor:
    if placement[0] == "R":
        return pieces[0]
    dim = placement[1]
    nonempty = [p for p in pieces if p.numel() > 0 or p.shape[dim] > 0]
    out = torch.cat(list(nonempty) if nonempty else [pieces[0]], dim=dim)
    if full_dim_size >= 0 and out.shape[dim] > full_dim_size:  # padded even sharding
        out = out.narrow(dim, 0, full_dim_size)
    return out


def consolidate_key(values: List[Any], full_shape=None) -> torch.Tensor:
    """``values[r]`` is rank r's saved entry for one key (ranks in C-order over the mesh)."""
    local0, placements, mesh_shape = _describe(values[0])
    if placements is None:
        return local0
    locals_ = [_describe(v)[0] for v in values]
    n = 1
    for s in mesh_shape:
        n *= s
    if len(locals_) != n:
        raise ValueError(f"expected {n} shards for mesh {mesh_shape}, got {len(locals_)}")
    # fold innermost mesh axis first; ranks are laid out C-order over the mesh
    cur = locals_
    for axis in range(len(mesh_shape) - 1, -1, -1):
        size = mesh_shape[axis]
        nxt = []
        for g in range(0, len(cur), size):
            dim_size = -1
            if full_shape is not None and placements[axis][0] == "S":
                # only trim on the outermost use of this tensor dim
                outer_same = any(placements[a] == placements[axis] for a in range(axis))
                if not outer_same:
                    dim_size = full_shape[placements[axis][1]]
            nxt.append(fold_axis(cur[g : g + size], placements[axis], dim_size))
        cur = nxt
    assert len(cur) == 1
    return cur[0]


def consolidate(shards: List[Dict[str, Any]]) -> Dict[str, torch.Tensor]:
    """Merge ``shards[r]`` (rank r's state dict) into one full state dict."""
    out: Dict[str, torch.Tensor] = {}
    for key in shards[0].keys():
        vals = [sd[key] for sd in shards]
        full_shape = tuple(vals[0].shape) if hasattr(vals[0], "placements") else None
        out[key] = consolidate_key(vals, full_shape)
    return out
