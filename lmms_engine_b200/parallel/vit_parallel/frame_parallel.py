"""ViT frame parallelism over the flattened dp x cp group: patches of whole frames travel to
the rank the LPT plan assigns, the tower runs on a balanced load, merged features travel back
(reference: src/lmms_engine/models/qwen3_vl/qwen3_vl_vit_ops.py:22-242,
src/lmms_engine/parallel/vit_parallel/frame_parallel.py:12-39)."""
from __future__ import annotations

from typing import List

import torch
import torch.distributed as dist

from ..expert_parallel import _AllToAllRows
from .balance import plan_frame_exchange


def balanced_vit_forward(tower, patches: torch.Tensor, grid_thw: torch.Tensor, group, slack: float = 0.25):
    """Run ``tower(patches, grid)`` with frames balanced across ``group``.  Returns the merged
    features of THIS rank's own frames, in their original order (deepstack lists included)."""
    n, me = dist.get_world_size(group), dist.get_rank(group)
    grid = [tuple(int(x) for x in g) for g in grid_thw.tolist()]
    # treat every temporal step as a frame so that long videos can be split
    frames = [(1, h, w) for t, h, w in grid for _ in range(t)]
    mine = [h * w for _, h, w in frames]
    gathered: List[List[int]] = [None] * n
    dist.all_gather_object(gathered, mine, group=group)
    shapes: List[list] = [None] * n
    dist.all_gather_object(shapes, frames, group=group)
    owner, send, _ = plan_frame_exchange(gathered, slack)
    # order my patches by destination rank (stable), remember the inverse
    starts = [0]
    for c in mine:
        starts.append(starts[-1] + c)
    order = sorted(range(len(mine)), key=lambda i: (owner[me][i], i))
    idx = torch.cat([torch.arange(starts[i], starts[i + 1]) for i in order]) if order else torch.zeros(0, dtype=torch.long)
    idx = idx.to(patches.device)
    send_p = [send[me][d] for d in range(n)]
    recv_p = [send[s][me] for s in range(n)]
    got = _AllToAllRows.apply(patches.index_select(0, idx), send_p, recv_p, group)
    recv_frames = [shapes[s][i] for s in range(n) for i in sorted(range(len(gathered[s])), key=lambda j: (owner[s][j], j))
                   if owner[s][i] == me]
    unit = tower.cfg.spatial_merge_size ** 2
    n_deep = len(getattr(tower, "deepstack_merger_list", []) or [])
    if recv_frames:
        out = tower(got, torch.tensor(recv_frames, dtype=torch.long, device=patches.device))
        feats, deep = out if isinstance(out, tuple) else (out, None)
    else:
        # nothing assigned to this rank: still contribute (empty) rows so that the exchange and the
        # autograd graph have the same shape everywhere
        width = tower.cfg.out_hidden_size
        if any(hasattr(p, "to_local") for p in tower.parameters()):
            raise RuntimeError("ViT frame balancing found a rank without frames while the tower's parameters are sharded "
                               "(FSDP2): a sharded tower must run on every rank; turn vit_frame_parallel off for this layout")
        feats = got.new_zeros((0, width)) + 0.0 * sum(p.sum() for p in tower.parameters() if p.requires_grad).to(got.dtype)
        deep = [feats for _ in range(n_deep)] if n_deep else None
    back_send = [c // unit for c in recv_p]
    back_recv = [c // unit for c in send_p]

    def go_home(t):
        home = _AllToAllRows.apply(t, back_send, back_recv, group)
        # undo the by-destination ordering at merged-token granularity
        m_starts = [0]
        for i in order:
            m_starts.append(m_starts[-1] + mine[i] // unit)
        pieces = [None] * len(mine)
        for k, i in enumerate(order):
            pieces[i] = home[m_starts[k]:m_starts[k + 1]]
        return torch.cat(pieces) if pieces else home

    feats = go_home(feats)
    if deep is not None:
        deep = [go_home(d) for d in deep]
        return feats, deep
    return feats


# ------------------------------------------------------------------ a sequence-parallel group shares one sample
class _GatherRows(torch.autograd.Function):
    """All-gather of row blocks of different heights (``counts[r]`` rows from rank r), rank after rank.  Backward sums
    every rank's gradient of this rank's rows (reduce-scatter; an all-reduce on back ends without one)."""

    @staticmethod
    def forward(ctx, x, counts, group):
        n, me = dist.get_world_size(group), dist.get_rank(group)
        mx = max(max(counts), 1)
        pad = x.new_zeros((mx,) + tuple(x.shape[1:]))
        pad[: x.shape[0]] = x
        out = x.new_empty((n * mx,) + tuple(x.shape[1:]))
        dist.all_gather_into_tensor(out, pad.contiguous(), group=group)
        ctx.meta = (list(counts), group, n, me, mx)
        return torch.cat([out[r * mx: r * mx + counts[r]] for r in range(n)], 0)

    @staticmethod
    def backward(ctx, g):
        counts, group, n, me, mx = ctx.meta
        buf = g.new_zeros((n * mx,) + tuple(g.shape[1:]))
        at = 0
        for r in range(n):
            buf[r * mx: r * mx + counts[r]] = g[at: at + counts[r]]
            at += counts[r]
        if dist.get_backend(group) == "nccl":
            mine = g.new_empty((mx,) + tuple(g.shape[1:]))
            dist.reduce_scatter_tensor(mine, buf, group=group)
        else:
            dist.all_reduce(buf, group=group)
            mine = buf[me * mx: (me + 1) * mx]
        return mine[: counts[me]], None, None


def deal_frames(sizes: List[int], n: int) -> List[int]:
    """Owner rank of every frame: largest first onto the least loaded rank (ties: lowest rank), the same on every rank."""
    load, owner = [0] * n, [0] * len(sizes)
    for i in sorted(range(len(sizes)), key=lambda j: (-sizes[j], j)):
        r = min(range(n), key=lambda q: (load[q], q))
        owner[i] = r
        load[r] += sizes[i]
    return owner


def sp_sharded_vit_forward(tower, patches: torch.Tensor, grid_thw: torch.Tensor, sp_group, run=None, always_run: bool = False):
    """The ranks of a sequence-parallel group hold the SAME sample, so running the tower on every rank repeats the work
    ``sp`` times and keeps ``sp`` copies of its activations.  Here every rank runs the tower on its share of the frames
    (dealt by size) and the merged features are all-gathered back into frame order; the gather's backward sums the
    ranks' gradients of a frame's features, which the owner back-propagates.  ``run(patches, grid)`` replaces the plain
    tower call (the frame balancing across the data-parallel ranks, with ``always_run``).  The reference splits the deepstack features
    per sequence-parallel rank but runs its tower on every rank (src/lmms_engine/models/qwen3_vl/qwen3_vl_ops.py:47-142)."""
    n, me = dist.get_world_size(sp_group), dist.get_rank(sp_group)
    run = run if run is not None else tower
    frames = [(1, int(h), int(w)) for t, h, w in grid_thw.tolist() for _ in range(int(t))]
    sizes = [h * w for _, h, w in frames]
    owner = deal_frames(sizes, n)
    starts = [0]
    for c in sizes:
        starts.append(starts[-1] + c)
    mine = [i for i in range(len(frames)) if owner[i] == me]
    unit = tower.cfg.spatial_merge_size ** 2
    n_deep = len(getattr(tower, "deepstack_merger_list", []) or [])
    if mine or always_run:  # ``always_run``: ``run`` holds collectives of its own that every rank must enter
        rows = (torch.cat([torch.arange(starts[i], starts[i + 1]) for i in mine]) if mine else torch.zeros(0, dtype=torch.long)).to(patches.device)
        sub_grid = torch.tensor([frames[i] for i in mine], dtype=torch.long, device=patches.device).reshape(-1, 3)
        out = run(patches.index_select(0, rows), sub_grid)
        feats, deep = out if isinstance(out, tuple) else (out, None)
    elif frames and any(hasattr(p, "to_local") for p in tower.parameters()):
        # the tower's parameters are held in shards (FSDP2): its gathers and gradient reductions are collectives that every
        # rank must enter, so a rank without a frame runs the smallest frame of the sample and keeps none of its rows
        # (the empty slices stay in the graph, which sends zero gradients through the wrapper's reductions)
        i = min(range(len(frames)), key=lambda j: (sizes[j], j))
        rows = torch.arange(starts[i], starts[i + 1], device=patches.device)
        out = run(patches.index_select(0, rows), torch.tensor([frames[i]], dtype=torch.long, device=patches.device))
        feats, deep = out if isinstance(out, tuple) else (out, None)
        feats, deep = feats[:0], ([d[:0] for d in deep] if deep is not None else None)
    else:
        feats = patches.new_zeros((0, tower.cfg.out_hidden_size)) + 0.0 * sum(p.sum() for p in tower.parameters() if p.requires_grad).to(patches.dtype)
        deep = [feats for _ in range(n_deep)] if n_deep else None
    counts = [sum(sizes[i] for i in range(len(frames)) if owner[i] == r) // unit for r in range(n)]
    # rank-major order of the gathered rows -> frame order
    merged = [c // unit for c in sizes]
    at, where = 0, [0] * len(frames)
    for r in range(n):
        for i in range(len(frames)):
            if owner[i] == r:
                where[i] = at
                at += merged[i]
    back = torch.cat([torch.arange(where[i], where[i] + merged[i]) for i in range(len(frames))]).to(patches.device) if frames else None

    def home(t):
        full = _GatherRows.apply(t, counts, sp_group)
        return full.index_select(0, back) if back is not None else full

    feats = home(feats)
    if deep is not None:
        return feats, [home(d) for d in deep]
    return feats
