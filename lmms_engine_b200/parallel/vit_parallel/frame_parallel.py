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
