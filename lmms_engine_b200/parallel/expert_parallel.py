"""Expert parallelism: experts are sharded over the ``ep`` group (``E / ep`` consecutive
experts per rank); tokens travel to the rank that owns their expert and back.

``ExpertParallel`` is attached to every sparse block (``SparseMoeBlock.ep``).  Layout:

* sender: the local permutation already orders rows by GLOBAL expert id with every expert's
  segment padded to the 128-row GEMM tile, so the rows bound for rank r are one contiguous
  block and tile alignment survives the exchange;
* exchange: counts all-gather, then one all-to-all of rows (and its mirror image back);
* receiver: blocks arrive source-major; one index-select regroups them expert-major so that
  each local expert owns one contiguous row range for the grouped GEMMs.

This module is the torch.distributed (NCCL / gloo) implementation and needs one host
read of the count matrix per layer, exactly like the reference
(src/lmms_engine/parallel/expert_parallel/utils.py:11-77,
src/lmms_engine/parallel/qwen3_moe/style.py:48-84).  ``apply_expert_parallel`` shards the
stacked expert parameters on dim 0 like the reference's partition function
(src/lmms_engine/parallel/qwen3_moe/style.py:92-113).
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from ..ops import moe as moe_ops

TILE = moe_ops.TILE


class _AllToAllRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, in_splits, out_splits, group):
        ctx.cfg = (in_splits, out_splits, group)
        out = x.new_empty((sum(out_splits),) + tuple(x.shape[1:]))
        dist.all_to_all_single(out, x.contiguous(), output_split_sizes=out_splits, input_split_sizes=in_splits, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        in_splits, out_splits, group = ctx.cfg
        out = g.new_empty((sum(in_splits),) + tuple(g.shape[1:]))
        dist.all_to_all_single(out, g.contiguous(), output_split_sizes=in_splits, input_split_sizes=out_splits, group=group)
        return out, None, None, None


def _pad(n: int) -> int:
    return (n + TILE - 1) // TILE * TILE


class ExpertParallel:
    def __init__(self, group, num_experts: int):
        self.group = group
        self.ep = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if num_experts % self.ep:
            raise ValueError(f"num_experts ({num_experts}) must be divisible by ep_degree ({self.ep})")
        self.E = num_experts
        self.El = num_experts // self.ep

    def plan(self, counts: torch.Tensor):
        """Exchange counts and derive every split size and index table (one host read)."""
        all_counts = torch.empty(self.ep * self.E, dtype=counts.dtype, device=counts.device)
        dist.all_gather_into_tensor(all_counts, counts.contiguous(), group=self.group)
        C = all_counts.view(self.ep, self.E).cpu().tolist()  # C[s][e]
        P = [[_pad(c) for c in row] for row in C]
        me, El = self.rank, self.El
        in_splits = [sum(P[me][r * El:(r + 1) * El]) for r in range(self.ep)]
        out_splits = [sum(P[s][me * El:(me + 1) * El]) for s in range(self.ep)]
        # received layout is source-major: [s][e_local][segment]; regroup to expert-major
        src_off = [0]
        for s in range(self.ep):
            src_off.append(src_off[-1] + out_splits[s])
        regroup: List[torch.Tensor] = []
        expert_start = [0]
        for el in range(El):
            e = me * El + el
            for s in range(self.ep):
                seg0 = src_off[s] + sum(P[s][me * El:e])
                regroup.append(torch.arange(seg0, seg0 + P[s][e]))
            expert_start.append(expert_start[-1] + sum(P[s][e] for s in range(self.ep)))
        dev = counts.device
        idx = torch.cat(regroup).to(dev) if regroup else torch.zeros(0, dtype=torch.long, device=dev)
        rows = expert_start[-1]
        tile_expert = torch.repeat_interleave(
            torch.arange(El, dtype=torch.int32),
            torch.tensor([(expert_start[i + 1] - expert_start[i]) // TILE for i in range(El)]),
        ).to(dev)
        local = moe_ops.Permutation(
            row_of=None, token_of_row=None, weight_of_row=None, tile_expert=tile_expert,
            expert_start=torch.tensor(expert_start, dtype=torch.int32, device=dev), rows=rows, n_experts=El)
        inverse = torch.empty_like(idx)
        inverse[idx] = torch.arange(idx.numel(), device=dev)
        return in_splits, out_splits, idx, inverse, local

    def __call__(self, x, idx, w, counts, experts) -> torch.Tensor:
        perm = moe_ops.build_permutation(idx, w, counts)  # by global expert id
        xp = moe_ops.dispatch(x, perm)
        in_splits, out_splits, regroup, inverse, local = self.plan(counts)
        used = sum(in_splits)
        recv = _AllToAllRows.apply(xp[:used], in_splits, out_splits, self.group)
        grouped = recv.index_select(0, regroup)
        yp = experts(grouped, local)
        back = _AllToAllRows.apply(yp.index_select(0, inverse), out_splits, in_splits, self.group)
        if used < perm.rows:
            back = torch.cat([back, back.new_zeros((perm.rows - used, back.shape[1]))], 0)
        return moe_ops.combine(back, w, perm)


_PEER_DISPATCHERS = {}


def make_dispatcher(group, num_experts: int, device):
    """One dispatcher per (group, expert count): over peer memory when the group's ranks can map each
    other's memory (``csrc/ep_comm.cu``), NCCL / gloo all-to-all otherwise."""
    from . import fused_ops

    key = (id(group), num_experts)
    if key not in _PEER_DISPATCHERS:
        ep = None
        if torch.device(device).type == "cuda" and fused_ops.peer_memory_ok(group):
            from .peer_expert_parallel import PeerExpertParallel

            ep = fused_ops.agree_or_none(
                lambda: PeerExpertParallel(group, num_experts, torch.device("cuda", torch.cuda.current_device())), group,
                "expert parallelism over peer memory")
        _PEER_DISPATCHERS[key] = ep if ep is not None else ExpertParallel(group, num_experts)
    return _PEER_DISPATCHERS[key]


def _local_tensor(p):
    """Expert parameters may be DTensors sharded over the ep mesh: compute on the local shard."""
    if hasattr(p, "to_local"):
        return p.to_local()
    return p


def apply_expert_parallel(model: nn.Module, ep_mesh, ep_group) -> None:
    """Shard every ``Experts`` module's stacked parameters on dim 0 over the ep mesh and attach
    the dispatcher to its sparse block."""
    from torch.distributed.tensor import Shard, distribute_tensor

    from ..models.moe_lm import SparseMoeBlock

    for block in model.modules():
        if not isinstance(block, SparseMoeBlock):
            continue
        ex = block.experts
        for name in ("gate_up_proj", "down_proj"):
            p = getattr(ex, name)
            setattr(ex, name, nn.Parameter(distribute_tensor(p.data, ep_mesh, [Shard(0)]), requires_grad=p.requires_grad))
        block.ep = make_dispatcher(ep_group, ex.num_experts, p.device)
