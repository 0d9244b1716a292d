"""Mixture-of-experts operators: router, deterministic sort-free permutation, grouped expert
MLP on the tcgen05 grouped GEMM, weighted combine, load-balancing loss.

Pipeline of one sparse block (no host synchronisation anywhere; buffers are sized for the
worst case ``T*k + E*127`` rows, rounded to the 128-row GEMM tile):

    probs, idx, w, counts = router_topk(logits)
    meta = build_permutation(idx, w, counts)             # row ranges padded per expert
    xp   = dispatch(x, meta)                              # gather into expert-major rows
    yp   = grouped_mlp(xp, gate_up_proj, down_proj, meta) # 2 grouped GEMMs, SwiGLU epilogue
    y    = combine(yp, meta, w)                           # sum_j w[t,j] * yp[row(t,j)]

Reference behaviour: src/lmms_engine/models/qwen3_moe/qwen3_moe_ops.py:257-322 (softmax ->
top-k -> renorm -> histc -> argsort -> per-expert Python loop -> scatter_add) and the HF
``load_balancing_loss_func`` used at src/lmms_engine/models/qwen3_moe/qwen3_moe_liger.py:146-157.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

from . import _cuda

_cuda.register("b200_moe_router", "moe", "pippppiiiiis")
_cuda.register("b200_moe_permute", "moe", "ppppppppiiils")
_cuda.register("b200_moe_debug_bad_index", "moe", "")
_cuda.register("b200_moe_combine", "moe", "ppppiii" + "lps")
_cuda.register("b200_moe_combine_bwd_src", "moe", "pppplilps")
_cuda.register("b200_moe_combine_bwd_w", "moe", "pppplii" + "lps")
_cuda.register("b200_moe_row_scale_dot", "moe", "plpppplis")
_cuda.register("b200_swiglu_cat_fwd", "moe", "pplis")
_cuda.register("b200_swiglu_cat_bwd", "moe", "pplis")
_cuda.register("b200_gemm_grouped_bf16", "gemm_sm100", "ppppiiiiiiips")
_cuda.register("b200_gemm_grouped_swiglu_bf16", "gemm_sm100", "pppppiiiiips")
_cuda.register("b200_gemm_grouped_wgrad_bf16", "gemm_sm100", "ppppiiiiiips")

TILE = 128


# ------------------------------------------------------------------------------ router
def router_ref(logits: torch.Tensor, k: int, renorm: bool):
    probs = torch.softmax(logits.float(), dim=-1)
    # ties resolve to the lower expert index, like the kernel
    w, idx = torch.topk(probs, k, dim=-1)
    if renorm:
        w = w / w.sum(-1, keepdim=True)
    counts = torch.bincount(idx.flatten(), minlength=logits.shape[-1]).to(torch.int32)
    return probs, idx.to(torch.int32), w, counts


class _RouterFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, k, renorm):
        T, E = logits.shape
        logits = logits.contiguous()
        dev = logits.device
        probs = torch.empty((T, E), dtype=torch.float32, device=dev)
        idx = torch.empty((T, k), dtype=torch.int32, device=dev)
        w = torch.empty((T, k), dtype=torch.float32, device=dev)
        counts = torch.empty(E, dtype=torch.int32, device=dev)
        _cuda.call("b200_moe_router", logits.data_ptr(), int(logits.dtype == torch.float32), probs.data_ptr(),
                   idx.data_ptr(), w.data_ptr(), counts.data_ptr(), T, E, k, int(renorm), 1, _cuda.stream())
        ctx.save_for_backward(probs, idx, w)
        ctx.cfg = (renorm, logits.dtype)
        ctx.mark_non_differentiable(idx, counts)
        return probs, idx, w, counts

    @staticmethod
    def backward(ctx, dprobs, _didx, dw, _dcounts):
        probs, idx, w = ctx.saved_tensors
        renorm, dtype = ctx.cfg
        lidx = idx.long()
        dp = dprobs.clone() if dprobs is not None else torch.zeros_like(probs)
        if dw is not None:
            if renorm:
                sel = probs.gather(1, lidx)
                s = sel.sum(-1, keepdim=True)
                dsel = (dw - (dw * w).sum(-1, keepdim=True)) / s
            else:
                dsel = dw
            dp.scatter_add_(1, lidx, dsel)
        dlogits = probs * (dp - (dp * probs).sum(-1, keepdim=True))
        return dlogits.to(dtype), None, None


def router_topk(logits: torch.Tensor, k: int, renorm: bool = True):
    """softmax -> top-k (-> renormalise).  Returns ``probs [T,E] fp32, idx [T,k] int32,
    weights [T,k] fp32, counts [E] int32``."""
    E = logits.shape[-1]
    if logits.is_cuda and E % 32 == 0 and E <= 256 and k <= 16 and logits.dtype in (torch.bfloat16, torch.float32):
        return _RouterFn.apply(logits, k, renorm)
    return router_ref(logits, k, renorm)


# ------------------------------------------------------------------------------ permutation
@dataclass
class Permutation:
    row_of: torch.Tensor  # int32 [T, k]   destination row of every (token, slot)
    token_of_row: torch.Tensor  # int64 [rows]   source token or -1 (padding)
    weight_of_row: torch.Tensor  # fp32  [rows]
    tile_expert: torch.Tensor  # int32 [rows/128]  expert of every 128-row tile or -1
    expert_start: torch.Tensor  # int32 [E+1]   padded row range of every expert
    rows: int  # worst-case number of rows (multiple of 128)
    n_experts: int


def max_rows(T: int, k: int, E: int) -> int:
    return (T * k + E * (TILE - 1) + TILE - 1) // TILE * TILE


def build_permutation(idx: torch.Tensor, w: torch.Tensor, counts: torch.Tensor) -> Permutation:
    T, k = idx.shape
    E = counts.numel()
    rows = max_rows(T, k, E)
    dev = idx.device
    if idx.is_cuda:
        expert_start = torch.empty(E + 1, dtype=torch.int32, device=dev)
        tile_expert = torch.empty(rows // TILE, dtype=torch.int32, device=dev)
        row_of = torch.empty((T, k), dtype=torch.int32, device=dev)
        token_of_row = torch.empty(rows, dtype=torch.int64, device=dev)
        weight_of_row = torch.empty(rows, dtype=torch.float32, device=dev)
        _cuda.call("b200_moe_permute", idx.data_ptr(), w.detach().contiguous().data_ptr(), counts.data_ptr(),
                   expert_start.data_ptr(), tile_expert.data_ptr(), row_of.data_ptr(), token_of_row.data_ptr(),
                   weight_of_row.data_ptr(), T, E, k, rows, _cuda.stream())
        return Permutation(row_of, token_of_row, weight_of_row, tile_expert, expert_start, rows, E)
    # reference construction (same layout)
    padded = (counts.long() + TILE - 1) // TILE * TILE
    start = torch.zeros(E + 1, dtype=torch.long)
    start[1:] = torch.cumsum(padded, 0)
    flat_e = idx.long().flatten()
    order = torch.sort(flat_e, stable=True).indices
    sorted_e = flat_e[order]
    rank_in_e = torch.arange(order.numel()) - torch.searchsorted(sorted_e, sorted_e)
    dest = torch.empty(order.numel(), dtype=torch.long)
    dest[order] = start[sorted_e] + rank_in_e
    token_of_row = torch.full((rows,), -1, dtype=torch.int64)
    token_of_row[dest] = torch.arange(T).repeat_interleave(k)
    weight_of_row = torch.zeros(rows)
    weight_of_row[dest] = w.detach().flatten().float()
    tile_rows = torch.arange(rows // TILE) * TILE
    tile_expert = torch.searchsorted(start[1:], tile_rows, right=True)
    tile_expert = torch.where(tile_rows < start[E], tile_expert, torch.full_like(tile_expert, -1)).to(torch.int32)
    return Permutation(dest.view(T, k).to(torch.int32), token_of_row, weight_of_row, tile_expert, start.to(torch.int32), rows, E)


# ------------------------------------------------------------------------------ dispatch / combine
class _DispatchFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, perm: Permutation):
        H = x.shape[1]
        out = torch.empty((perm.rows, H), dtype=x.dtype, device=x.device)
        _cuda.call("b200_gather_rows", x.data_ptr(), perm.token_of_row.data_ptr(), out.data_ptr(), perm.rows, H, x.shape[0],
                   _cuda.status_word(x.device).data_ptr(), _cuda.stream())
        ctx.perm = perm
        ctx.T = x.shape[0]
        return out

    @staticmethod
    def backward(ctx, dout):
        perm = ctx.perm
        dout = dout.contiguous()
        H = dout.shape[1]
        k = perm.row_of.shape[1]
        dx = torch.empty((ctx.T, H), dtype=dout.dtype, device=dout.device)
        _cuda.call("b200_moe_combine", dout.data_ptr(), perm.row_of.data_ptr(), None, dx.data_ptr(), ctx.T, k, H, dout.shape[0],
                   _cuda.status_word(dout.device).data_ptr(), _cuda.stream())
        return dx, None


def dispatch(x: torch.Tensor, perm: Permutation) -> torch.Tensor:
    """``xp[row] = x[token_of_row[row]]`` (zero rows for padding)."""
    if x.is_cuda and x.dtype == torch.bfloat16 and x.shape[1] % 8 == 0:
        return _DispatchFn.apply(x.contiguous(), perm)
    safe = perm.token_of_row.clamp(min=0)
    out = x.index_select(0, safe)
    return out * (perm.token_of_row >= 0).unsqueeze(-1).to(out.dtype)


class _CombineFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, src, w, perm: Permutation):
        T, k = perm.row_of.shape
        H = src.shape[1]
        wf = w.float().contiguous()
        out = torch.empty((T, H), dtype=src.dtype, device=src.device)
        _cuda.call("b200_moe_combine", src.data_ptr(), perm.row_of.data_ptr(), wf.data_ptr(), out.data_ptr(), T, k, H, src.shape[0],
                   _cuda.status_word(src.device).data_ptr(), _cuda.stream())
        ctx.save_for_backward(src, wf)
        ctx.perm = perm
        ctx.wdtype = w.dtype
        return out

    @staticmethod
    def backward(ctx, dout):
        src, wf = ctx.saved_tensors
        perm = ctx.perm
        dout = dout.contiguous()
        T, k = perm.row_of.shape
        H = src.shape[1]
        dsrc = torch.empty_like(src) if src.shape[0] == perm.rows else torch.zeros_like(src)
        _cuda.call("b200_moe_combine_bwd_src", dout.data_ptr(), perm.token_of_row.data_ptr(), perm.weight_of_row.data_ptr(),
                   dsrc.data_ptr(), min(perm.rows, src.shape[0]), H, dout.shape[0], _cuda.status_word(src.device).data_ptr(), _cuda.stream())
        dw = torch.empty((T, k), dtype=torch.float32, device=src.device)
        _cuda.call("b200_moe_combine_bwd_w", dout.data_ptr(), src.data_ptr(), perm.row_of.data_ptr(), dw.data_ptr(), T * k, k, H, src.shape[0],
                   _cuda.status_word(src.device).data_ptr(), _cuda.stream())
        return dsrc, dw.to(ctx.wdtype), None


def combine(src: torch.Tensor, w: torch.Tensor, perm: Permutation) -> torch.Tensor:
    """``out[t] = sum_j w[t,j] * src[row_of[t,j]]``."""
    if src.is_cuda and src.dtype == torch.bfloat16 and src.shape[1] % 8 == 0:
        return _CombineFn.apply(src.contiguous(), w, perm)
    rows = src.index_select(0, perm.row_of.long().flatten()).view(*perm.row_of.shape, -1)
    return (rows.float() * w.float().unsqueeze(-1)).sum(1).to(src.dtype)


# ------------------------------------------------------------------------------ grouped expert MLP
def _grouped(a, w, perm, w_mn_major, n_out):
    rows, K = a.shape
    out = torch.empty((rows, n_out), dtype=a.dtype, device=a.device)
    st = _cuda.status_word(a.device)
    _cuda.call("b200_gemm_grouped_bf16", a.data_ptr(), w.data_ptr(), out.data_ptr(), perm.tile_expert.data_ptr(), rows,
               n_out, K, perm.n_experts, a.stride(0), out.stride(0), int(w_mn_major), st.data_ptr(), _cuda.stream())
    return out


def _wgrad(a, b, perm):
    rows, M = a.shape
    N = b.shape[1]
    E = perm.n_experts
    out = torch.empty((E, M, N), dtype=a.dtype, device=a.device)
    st = _cuda.status_word(a.device)
    _cuda.call("b200_gemm_grouped_wgrad_bf16", a.data_ptr(), b.data_ptr(), out.data_ptr(), perm.expert_start.data_ptr(),
               rows, M, N, E, a.stride(0), b.stride(0), st.data_ptr(), _cuda.stream())
    return out


class _GroupedMLPFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, xp, gate_up, down, perm: Permutation):
        rows, H = xp.shape
        E, two_i, _ = gate_up.shape
        inter = two_i // 2
        h = torch.empty((rows, inter), dtype=xp.dtype, device=xp.device)
        # unused tiles are never written by the kernels: keep them finite
        gu = torch.zeros((rows, two_i), dtype=xp.dtype, device=xp.device)
        st = _cuda.status_word(xp.device)
        _cuda.call("b200_gemm_grouped_swiglu_bf16", xp.data_ptr(), gate_up.data_ptr(), h.data_ptr(), gu.data_ptr(),
                   perm.tile_expert.data_ptr(), rows, inter, H, E, xp.stride(0), st.data_ptr(), _cuda.stream())
        yp = _grouped(h, down, perm, False, H)
        ctx.save_for_backward(xp, gate_up, down, gu)
        ctx.perm = perm
        return yp

    @staticmethod
    def backward(ctx, dyp):
        xp, gate_up, down, gu = ctx.saved_tensors
        perm = ctx.perm
        dyp = dyp.contiguous()
        rows, H = xp.shape
        inter = gu.shape[1] // 2
        h = torch.empty((rows, inter), dtype=xp.dtype, device=xp.device)
        _cuda.call("b200_swiglu_cat_fwd", gu.data_ptr(), h.data_ptr(), rows, inter, _cuda.stream())
        d_down = _wgrad(dyp, h, perm) if ctx.needs_input_grad[2] else None  # [E, H, I]
        dh = _grouped(dyp, down, perm, True, inter)  # dyp [rows,H] @ down[e] [H,I]
        _cuda.call("b200_swiglu_cat_bwd", dh.data_ptr(), gu.data_ptr(), rows, inter, _cuda.stream())  # gu <- [dg | du]
        d_gate_up = _wgrad(gu, xp, perm) if ctx.needs_input_grad[1] else None  # [E, 2I, H]
        dxp = _grouped(gu, gate_up, perm, True, H) if ctx.needs_input_grad[0] else None
        return dxp, d_gate_up, d_down, None


def grouped_mlp_ref(xp, gate_up, down, perm: Permutation):
    out = torch.zeros((xp.shape[0], down.shape[1]), dtype=xp.dtype, device=xp.device)
    start = perm.expert_start.tolist()
    inter = gate_up.shape[1] // 2
    for e in range(perm.n_experts):
        lo, hi = start[e], start[e + 1]
        if hi <= lo:
            continue
        gu = F.linear(xp[lo:hi], gate_up[e])
        h = F.silu(gu[:, :inter]) * gu[:, inter:]
        out[lo:hi] = F.linear(h, down[e])
    return out


def grouped_mlp(xp, gate_up, down, perm: Permutation) -> torch.Tensor:
    """Per-expert ``down(silu(x Wg^T) * (x Wu^T))`` over expert-major rows."""
    native = (xp.is_cuda and xp.dtype == torch.bfloat16 and gate_up.dtype == torch.bfloat16 and xp.shape[1] % 8 == 0
              and (gate_up.shape[1] // 2) % 8 == 0 and gate_up.is_contiguous() and down.is_contiguous())
    if native:
        return _GroupedMLPFn.apply(xp.contiguous(), gate_up, down, perm)
    return grouped_mlp_ref(xp, gate_up, down, perm)


# ------------------------------------------------------------------------------ aux loss
def load_balancing_loss(probs: torch.Tensor, counts: torch.Tensor, k: int) -> torch.Tensor:
    """``E * sum_e f_e * P_e`` with ``f_e`` the fraction of (token, slot) assignments per slot
    going to expert e (= counts_e / T) and ``P_e`` the mean router probability."""
    T, E = probs.shape
    f = counts.to(torch.float32) / max(T, 1)
    return E * (f * probs.mean(0)).sum()


def row_scale_dot(g: torch.Tensor, y: torch.Tensor, w: torch.Tensor, dot_out: torch.Tensor) -> torch.Tensor:
    """``d_y = w[:, None] * g`` (in ``y``'s dtype) and ``dot_out[r] = <g[r], y[r]>`` in one pass over ``g`` and ``y``: the
    expert side of the combine's backward when the gradient rows already sit next to their router weights."""
    rows, H = y.shape
    if g.is_cuda and g.dtype == torch.bfloat16 and y.dtype == torch.bfloat16 and H % 8 == 0 and g.stride(1) == 1 and g.stride(0) % 8 == 0:
        d_y = torch.empty_like(y)
        _cuda.call("b200_moe_row_scale_dot", g.data_ptr(), g.stride(0), y.contiguous().data_ptr(), w.data_ptr(), d_y.data_ptr(),
                   dot_out.data_ptr(), rows, H, _cuda.stream())
        return d_y
    gf = g.float()
    dot_out.copy_((gf * y.float()).sum(1))
    return (gf * w.unsqueeze(1)).to(y.dtype)
