"""Autograd layers built on the GEMMs with fused collectives (``fused_comm``).

* ``column_linear`` / ``row_linear``: the two projections of sequence-parallel tensor parallelism.
  Forward of the first is all-gather -> GEMM, its input gradient is GEMM -> reduce-scatter (which
  also re-gathers the input for the weight gradient); the second is the mirror image.
* ``ulysses_qkv`` / ``ulysses_out``: the projections on either side of Ulysses attention.  The QKV
  GEMM writes each head's columns straight into the head-sharded layout on the rank that owns the
  head; the output projection gathers the attention output of its tokens from all ranks before
  its tiles; the backward passes use the opposite kernels.

``context_for(group)`` decides whether a group can use them: CUDA, NCCL, at most eight ranks, all on
one host (peer-mapped memory), and not disabled with ``LMMS_B200_FUSED_COMM=0``.  Otherwise the
callers keep the NCCL collectives of ``tp_ops`` / ``sequence_parallel.ulysses`` around plain GEMMs,
which is also what the reference does (src/lmms_engine/parallel/sequence_parallel/ulysses.py:101-330).
"""
from __future__ import annotations

import os
import socket
from typing import Dict, Optional

import torch
import torch.distributed as dist

from ..ops import gemm as gemm_ops
from . import tp_ops
from .fused_comm import FusedComm, HeadRoute, out_head_route, qkv_head_route, qkv_kb_sources

_CONTEXTS: Dict[int, Optional[FusedComm]] = {}


def peer_memory_ok(group) -> bool:
    """Can the ranks of ``group`` map each other's memory?  CUDA, NCCL, at most eight ranks, one host,
    and not disabled with ``LMMS_B200_FUSED_COMM=0``.  Collective on first use per group."""
    ok = (
        os.environ.get("LMMS_B200_FUSED_COMM", "1") != "0"
        and torch.cuda.is_available()
        and dist.is_initialized()
        and dist.get_backend(group) == "nccl"
        and dist.get_world_size(group) <= 8
    )
    if ok:
        hosts = [None] * dist.get_world_size(group)
        dist.all_gather_object(hosts, socket.gethostname(), group=group)
        ok = len(set(hosts)) == 1
    return ok


def context_for(group) -> Optional[FusedComm]:
    """The group's fused-collective context, created on first use (collectively), or None."""
    key = id(group)
    if key in _CONTEXTS:
        return _CONTEXTS[key]
    fc = None
    if peer_memory_ok(group):
        fc = agree_or_none(lambda: FusedComm(group, torch.device("cuda", torch.cuda.current_device())), group,
                           "fused collectives")
        if fc is not None:
            fc._routes = {}
    _CONTEXTS[key] = fc
    return fc


def agree_or_none(build, group, what: str):
    """Run ``build()`` on every rank of ``group``; keep the result only if it succeeded everywhere, so that
    a machine without peer access falls back to NCCL on all ranks together instead of splitting the group."""
    obj, err = None, None
    try:
        obj = build()
    except Exception as e:  # symmetric-memory allocation / rendezvous not available
        err = e
    flag = torch.tensor([1 if obj is not None else 0], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
    if int(flag.item()) == 0:
        if dist.get_rank(group) == 0:
            from ..utils.logging_utils import logger

            logger.warning(f"{what}: peer-mapped memory is not usable ({err}); using NCCL collectives")
        return None
    return obj


def _route(fc: FusedComm, kind: str, n_q: int, n_kv: int, D: int):
    k = (kind, n_q, n_kv, D)
    r = fc._routes.get(k)
    if r is None:
        if kind == "qkv":
            r = (qkv_head_route(n_q, n_kv, D, fc.world, fc.device), qkv_kb_sources(n_q, n_kv, D, fc.world, fc.device))
        else:
            r = (out_head_route(n_q, D, fc.world, fc.device), None)
        fc._routes[k] = r
    return r


def _c2(t: torch.Tensor, rows: int) -> torch.Tensor:
    t = t.reshape(rows, -1)
    return t if (t.stride(1) == 1 and t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0) else t.contiguous()


# ------------------------------------------------------------------------------- tensor parallel
def tp_supported(tokens_per_rank: int) -> bool:
    return tokens_per_rank % 128 == 0


class _ColumnLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias, fc):
        ctx.fc = fc
        ctx.save_for_backward(x, w)
        ctx.has_bias = bias is not None
        y, _ = fc.ag_gemm(x, w, bias=bias, key="ag_x")
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        fc = ctx.fc
        dy = _c2(dy, dy.shape[0])
        if fc.world <= fc.rs_fused_max_world:
            dx, xg = fc.gemm_rs(dy, w, b_mn=True, key="rs_dx", regather=(x, "regather_x"))
        else:
            dx = tp_ops._reduce_scatter(gemm_ops.matmul_nn(dy, w), fc.group)
            xg = tp_ops._all_gather(x, fc.group)
        dw = gemm_ops.matmul_tn(dy, xg)
        db = dy.sum(0, dtype=torch.float32).to(dy.dtype) if ctx.has_bias else None
        return dx, dw, db, None


class _RowLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, fc):
        ctx.fc = fc
        x = _c2(x, x.shape[0])
        ctx.save_for_backward(x, w)
        if fc.world <= fc.rs_fused_max_world:
            return fc.gemm_rs(x, w, key="rs_y")
        return tp_ops._reduce_scatter(gemm_ops.matmul_nt(x, w), fc.group)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        fc = ctx.fc
        dy = _c2(dy, dy.shape[0])
        dx, dyg = fc.ag_gemm(dy, w, b_mn=True, key="ag_dy")
        dw = gemm_ops.matmul_tn(dyg, x)
        return dx, dw, None


def column_linear(x, w, bias, fc: FusedComm):
    """``all_gather_rows(x) @ w^T + bias`` for a weight shard ``w [N/tp, K]``."""
    return _ColumnLinear.apply(x, w, bias, fc)


def row_linear(x, w, fc: FusedComm):
    """``reduce_scatter_rows(x @ w^T)`` for a weight shard ``w [N, K/tp]``."""
    return _RowLinear.apply(x, w, fc)


# ------------------------------------------------------------------------------- Ulysses
def ulysses_supported(n_q: int, n_kv: int, head_dim: int, world: int) -> bool:
    """Heads must split evenly (a replicated KV head would need its gradient summed over the
    replicas, which the scattering kernel does not do) and a head must be whole 64-column chunks."""
    return n_q % world == 0 and n_kv % world == 0 and head_dim % 64 == 0


class _UlyssesQKV(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias, fc, n_q, n_kv, D, layer):
        route, _ = _route(fc, "qkv", n_q, n_kv, D)
        x = _c2(x, x.shape[0])
        out = fc.gemm_a2a(x, w, route, bias=bias, key=("qkv", layer))
        ctx.fc, ctx.meta, ctx.has_bias = fc, (n_q, n_kv, D), bias is not None
        ctx.save_for_backward(x, w)
        T = out.shape[0]
        hq, hkv = n_q // fc.world, n_kv // fc.world
        q = out[:, : hq * D].view(T, hq, D)
        k = out[:, hq * D : (hq + hkv) * D].view(T, hkv, D)
        v = out[:, (hq + hkv) * D :].view(T, hkv, D)
        return q, k, v

    @staticmethod
    def backward(ctx, dq, dk, dv):
        x, w = ctx.saved_tensors
        fc = ctx.fc
        n_q, n_kv, D = ctx.meta
        hq, hkv = n_q // fc.world, n_kv // fc.world
        T = dq.shape[0]
        _, kb = _route(fc, "qkv", n_q, n_kv, D)
        parts = [(_c2(dq, T), fc.rank * hq * D), (_c2(dk, T), n_q * D + fc.rank * hkv * D),
                 (_c2(dv, T), (n_q + n_kv) * D + fc.rank * hkv * D)]
        dx, g = fc.a2a_gemm(parts, w, (n_q + 2 * n_kv) * D, kb_src=kb, b_mn=True, key="dqkv", k_rot=fc.rank * hq * D // 64)
        dw = gemm_ops.matmul_tn(g, x)
        db = g.sum(0, dtype=torch.float32).to(g.dtype) if ctx.has_bias else None
        return dx, dw, db, None, None, None, None, None


class _UlyssesOut(torch.autograd.Function):
    @staticmethod
    def forward(ctx, o, w, fc, n_q, D, layer):
        T = o.shape[0]
        hq = n_q // fc.world
        o2 = _c2(o, T)
        # the gathered attention output stays in this layer's own buffer until its backward pass
        y, g = fc.a2a_gemm([(o2, fc.rank * hq * D)], w, n_q * D, key=("o", layer), k_rot=fc.rank * hq * D // 64, rotate=False)
        ctx.fc, ctx.meta = fc, (n_q, D, T)
        ctx.save_for_backward(g, w)
        return y

    @staticmethod
    def backward(ctx, dy):
        g, w = ctx.saved_tensors
        fc = ctx.fc
        n_q, D, T = ctx.meta
        hq = n_q // fc.world
        route, _ = _route(fc, "out", n_q, 0, D)
        dy = _c2(dy, dy.shape[0])
        # attention backward of this layer consumes the buffer before any rank can reach the next
        # layer's call: the gradient all-to-all of the QKV projection in between needs every rank
        do = fc.gemm_a2a(dy, w, route, b_mn=True, key="dao")
        dw = gemm_ops.matmul_tn(dy, g)
        return do.view(T, hq, D), dw, None, None, None, None


def ulysses_qkv(x, w, bias, fc: FusedComm, n_q: int, n_kv: int, head_dim: int, layer: int):
    """QKV projection of my ``T/n`` tokens, returned head-sharded over all ``T`` tokens."""
    return _UlyssesQKV.apply(x, w, bias, fc, n_q, n_kv, head_dim, layer)


def ulysses_out(o, w, fc: FusedComm, n_q: int, head_dim: int, layer: int):
    """Output projection: ``o [T, Hq/n, D]`` -> ``[T/n, hidden]``."""
    return _UlyssesOut.apply(o, w, fc, n_q, head_dim, layer)
