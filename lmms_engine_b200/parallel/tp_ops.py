"""Collectives of the sequence-parallel tensor-parallel regions, with autograd.

Between blocks the token stream is split over the tensor-parallel ranks; a column-parallel
projection is preceded by an all-gather of tokens and a row-parallel projection is followed by
a reduce-scatter, so activations are never replicated and the all-reduce of plain Megatron TP
(what the reference's DTensor Colwise/Rowwise plan with ``use_local_output`` performs,
src/lmms_engine/parallel/qwen3_vl/parallelize.py:58-69) splits into its two halves.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def _all_gather(x, group):
    n = dist.get_world_size(group)
    out = x.new_empty((n * x.shape[0],) + tuple(x.shape[1:]))
    dist.all_gather_into_tensor(out, x.contiguous(), group=group)
    return out


def _reduce_scatter(x, group):
    n = dist.get_world_size(group)
    out = x.new_empty((x.shape[0] // n,) + tuple(x.shape[1:]))
    try:
        dist.reduce_scatter_tensor(out, x.contiguous(), group=group)
    except (RuntimeError, NotImplementedError):  # backends without reduce-scatter (gloo): all-reduce + slice
        full = x.contiguous().clone()
        dist.all_reduce(full, group=group)
        r = dist.get_rank(group)
        out = full[r * out.shape[0]:(r + 1) * out.shape[0]].clone()
    return out


class _AllGatherTokens(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _all_gather(x, group)

    @staticmethod
    def backward(ctx, g):
        return _reduce_scatter(g, ctx.group), None


class _ReduceScatterTokens(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _reduce_scatter(x, group)

    @staticmethod
    def backward(ctx, g):
        return _all_gather(g, ctx.group), None


def all_gather_tokens(x: torch.Tensor, group) -> torch.Tensor:
    return _AllGatherTokens.apply(x, group)


def reduce_scatter_tokens(x: torch.Tensor, group) -> torch.Tensor:
    return _ReduceScatterTokens.apply(x, group)


@torch.no_grad()
def sync_replicated_grads(model: torch.nn.Module, group) -> None:
    """Sum over the tensor-parallel group the gradients of parameters that are replicated
    there (norms, embeddings, lm_head, router): each rank saw a different token slice."""
    for name, p in model.named_parameters():
        if p.grad is None or getattr(p, "_tp_sharded", False):
            continue
        g = p.grad
        if hasattr(g, "placements"):
            mesh_names = g.device_mesh.mesh_dim_names or ()
            if "tp" in mesh_names and any(pl.is_shard() for pl, nm in zip(g.placements, mesh_names) if nm == "tp"):
                continue
            g = g._local_tensor
        dist.all_reduce(g, group=group)
