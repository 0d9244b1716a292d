"""Ulysses sequence parallelism: sequence <-> head all-to-all around attention.

Each rank of the sequence-parallel ("cp") group holds a contiguous ``T/n`` slice of the
packed stream with all heads; attention runs on the full sequence with ``H/n`` heads.
Capabilities mirror src/lmms_engine/parallel/sequence_parallel/ulysses.py:101-469 (group
registry, pad-and-slice, Q/K/V and output all-to-alls with autograd, KV-head replication
when ``n_kv < n``, loss gather with the ``x n`` gradient scale), with these differences:

* one fused all-to-all moves q, k and v together instead of three list-based calls,
* query heads that do not divide the group (28 heads over 8 ranks) are padded per GQA
  group with zero heads whose outputs are dropped, so such models can run at that degree,
* the loss reduction all-reduces two scalars instead of gathering per-token losses.

The collective itself goes through ``all_to_all_single`` (NCCL over NVLink, or gloo).
"""
from __future__ import annotations

from typing import Any, Optional, Tuple

import torch
import torch.distributed as dist

_ULYSSES_GROUP = None


def set_ulysses_sequence_parallel_group(group) -> None:
    global _ULYSSES_GROUP
    _ULYSSES_GROUP = group


def get_ulysses_sequence_parallel_group():
    return _ULYSSES_GROUP


def group_size(group) -> int:
    if group is None:
        return 1
    return dist.get_world_size(group)


def get_ulysses_sequence_parallel_world_size(group=None) -> int:
    return group_size(group if group is not None else _ULYSSES_GROUP)


def get_ulysses_sequence_parallel_rank(group=None) -> int:
    group = group if group is not None else _ULYSSES_GROUP
    return dist.get_rank(group) if group is not None else 0


def pad_to_multiple(x: torch.Tensor, n: int, value, dim: int = 0) -> torch.Tensor:
    """Right-pad ``dim`` (the token axis; the last axis for ``[3, T]`` positions) to a multiple of n."""
    if x.dim() == 2 and x.shape[0] == 3 and dim == 0 and x.dtype in (torch.int64, torch.int32):
        dim = 1
    pad = (-x.shape[dim]) % n
    if pad == 0:
        return x
    shape = list(x.shape)
    shape[dim] = pad
    return torch.cat([x, x.new_full(shape, value)], dim)


def slice_for_rank(x: torch.Tensor, group, dim: int = 0) -> torch.Tensor:
    n, r = group_size(group), dist.get_rank(group)
    if x.dim() == 2 and x.shape[0] == 3 and dim == 0 and x.dtype in (torch.int64, torch.int32):
        dim = 1
    chunk = x.shape[dim] // n
    return x.narrow(dim, r * chunk, chunk)


def ulysses_pad_and_slice_inputs(input_ids, position_ids=None, sp_size: Optional[int] = None, group=None):
    """Pad the flat stream to a multiple of the group size and keep this rank's slice."""
    group = group if group is not None else _ULYSSES_GROUP
    n = sp_size or group_size(group)
    pad = (-input_ids.shape[-1]) % n
    ids = slice_for_rank(pad_to_multiple(input_ids, n, 0, dim=input_ids.dim() - 1), group, dim=input_ids.dim() - 1)
    pos = None
    if position_ids is not None:
        pos = slice_for_rank(pad_to_multiple(position_ids, n, 0, dim=position_ids.dim() - 1), group, dim=position_ids.dim() - 1)
    return ids, pos, pad


def _a2a(x: torch.Tensor, group) -> torch.Tensor:
    """``x [n, ...]`` -> ``y [n, ...]`` with ``y[r] = (x of rank r)[my_rank]``."""
    out = torch.empty_like(x)
    try:
        dist.all_to_all_single(out, x.contiguous(), group=group)
    except RuntimeError:
        # backends without alltoall: emulate with an all-gather (test-only path)
        n = dist.get_world_size(group)
        bufs = [torch.empty_like(x) for _ in range(n)]
        dist.all_gather(bufs, x.contiguous(), group=group)
        me = dist.get_rank(group)
        out = torch.stack([b[me] for b in bufs], 0)
    return out


class _SeqToHead(torch.autograd.Function):
    """[T/n, H, D] (all heads, my tokens) -> [T, H/n, D] (my heads, all tokens)."""

    @staticmethod
    def forward(ctx, x, group):
        n = dist.get_world_size(group)
        Tl, H, D = x.shape
        ctx.group, ctx.shape = group, (Tl, H, D)
        send = x.view(Tl, n, H // n, D).permute(1, 0, 2, 3).contiguous()  # [n, Tl, H/n, D]
        recv = _a2a(send, group)
        return recv.view(n * Tl, H // n, D)

    @staticmethod
    def backward(ctx, g):
        group = ctx.group
        n = dist.get_world_size(group)
        Tl, H, D = ctx.shape
        send = g.contiguous().view(n, Tl, H // n, D)
        recv = _a2a(send, group)  # [n(head group), Tl, H/n, D]
        return recv.permute(1, 0, 2, 3).reshape(Tl, H, D), None


class _HeadToSeq(torch.autograd.Function):
    """[T, H/n, D] -> [T/n, H, D]."""

    @staticmethod
    def forward(ctx, x, group):
        n = dist.get_world_size(group)
        T, Hl, D = x.shape
        ctx.group, ctx.shape = group, (T, Hl, D)
        recv = _a2a(x.contiguous().view(n, T // n, Hl, D), group)
        return recv.permute(1, 0, 2, 3).reshape(T // n, n * Hl, D)

    @staticmethod
    def backward(ctx, g):
        group = ctx.group
        n = dist.get_world_size(group)
        T, Hl, D = ctx.shape
        send = g.view(T // n, n, Hl, D).permute(1, 0, 2, 3).contiguous()
        recv = _a2a(send, group)
        return recv.view(T, Hl, D), None


def gather_seq_scatter_heads(x: torch.Tensor, group=None) -> torch.Tensor:
    return _SeqToHead.apply(x, group if group is not None else _ULYSSES_GROUP)


def gather_heads_scatter_seq(x: torch.Tensor, group=None) -> torch.Tensor:
    return _HeadToSeq.apply(x, group if group is not None else _ULYSSES_GROUP)


def plan_heads(n_q: int, n_kv: int, n: int) -> Tuple[int, int, int]:
    """Head counts after padding / replication so that both divide ``n``.

    Returns ``(q_per_group_padded, kv_rep, n_kv_eff)``: every GQA group of ``n_q/n_kv``
    query heads is padded to ``q_per_group_padded`` heads and every KV head is repeated
    ``kv_rep`` times, so that ``n_kv * kv_rep`` and ``n_kv * q_per_group_padded`` are
    multiples of ``n`` and each rank ends up with whole (q heads, kv head) groups.
    """
    rep = 1
    while (n_kv * rep) % n != 0:
        rep += 1
    kv_eff = n_kv * rep
    group = n_q // n_kv
    # each replicated kv head serves group/rep query heads; pad group to a multiple of rep
    padded = ((group + rep - 1) // rep) * rep
    while (n_kv * padded) % n != 0:
        padded += rep
    return padded, rep, kv_eff


def seq_to_head_qkv(q, k, v, group):
    """Ulysses input exchange for q ``[T/n, Hq, D]`` and k, v ``[T/n, Hkv, D]`` in one all-to-all."""
    n = group_size(group)
    Tl, Hq, D = q.shape
    Hkv = k.shape[1]
    padded, rep, kv_eff = plan_heads(Hq, Hkv, n)
    gsz = Hq // Hkv
    if padded != gsz:
        qg = q.view(Tl, Hkv, gsz, D)
        qg = torch.cat([qg, qg.new_zeros(Tl, Hkv, padded - gsz, D)], 2)
        q = qg.reshape(Tl, Hkv * padded, D)
    if rep > 1:
        k = k.repeat_interleave(rep, 1)
        v = v.repeat_interleave(rep, 1)
    hq_l, hkv_l = q.shape[1] // n, kv_eff // n
    # interleave per destination rank: [q heads of rank g | k head(s) of g | v head(s) of g]
    fused = torch.cat(
        [q.view(Tl, n, hq_l, D), k.view(Tl, n, hkv_l, D), v.view(Tl, n, hkv_l, D)], 2
    ).reshape(Tl, n * (hq_l + 2 * hkv_l), D)
    out = _SeqToHead.apply(fused, group)  # [T, hq_l + 2 hkv_l, D]
    return out[:, :hq_l], out[:, hq_l : hq_l + hkv_l], out[:, hq_l + hkv_l :]


def head_to_seq(o: torch.Tensor, group, n_q: Optional[int] = None, n_kv: Optional[int] = None) -> torch.Tensor:
    """Inverse exchange for the attention output; drops padded query heads when told the true counts."""
    out = _HeadToSeq.apply(o, group)
    if n_q is not None and n_kv is not None and out.shape[1] != n_q:
        padded = out.shape[1] // n_kv
        gsz = n_q // n_kv
        out = out.view(out.shape[0], n_kv, padded, -1)[:, :, :gsz].reshape(out.shape[0], n_q, -1)
    return out


class _SPLossReduce(torch.autograd.Function):
    """Global token-weighted mean over the SP group.

    Backward hands each rank ``n / N_total``: gradients are later AVERAGED over the
    flattened dp x cp mesh by the sharded-data-parallel reduce-scatter, and every SP rank
    back-propagates only its own slice, so the factor ``n`` restores the full-sequence
    gradient (reference: ``Gather.backward``, ulysses.py:268-279).
    """

    @staticmethod
    def forward(ctx, local_sum, local_count, group, averaged):
        buf = torch.stack([local_sum.detach().float(), local_count.float()])
        dist.all_reduce(buf, group=group)
        total = buf[1].clamp(min=1.0)
        # `averaged`: the data-parallel reduction will divide by this group's size as well
        ctx.scale = (dist.get_world_size(group) if averaged else 1.0) / total
        return buf[0] / total

    @staticmethod
    def backward(ctx, g):
        return g * ctx.scale, None, None, None


def reduce_loss(per_token: torch.Tensor, valid: torch.Tensor, group, averaged_by_fsdp: bool = True) -> torch.Tensor:
    local_sum = (per_token * valid.to(per_token.dtype)).sum()
    return _SPLossReduce.apply(local_sum, valid.sum(), group, averaged_by_fsdp)


def calculate_seq_len_per_rank(cu_seqlens, sp_size: int, rank: int):
    """Document boundaries clipped to this rank's contiguous slice of the padded stream."""
    total = int(cu_seqlens[-1])
    total += (-total) % sp_size
    chunk = total // sp_size
    lo, hi = rank * chunk, (rank + 1) * chunk
    cuts = [min(max(int(c), lo), hi) - lo for c in cu_seqlens.tolist()]
    if cuts[-1] < chunk:
        cuts.append(chunk)
    out = [cuts[0]]
    for c in cuts[1:]:
        if c != out[-1]:
            out.append(c)
    if out[0] != 0:
        out.insert(0, 0)
    return out
