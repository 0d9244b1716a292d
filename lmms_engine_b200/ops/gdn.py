"""Chunked gated delta rule over a packed batch of documents.

Every document is padded to a multiple of 64 tokens and all chunks of all documents form one batch:
the in-chunk work (decay matrices, the unit-triangular solve, in-chunk attention) runs as batched ops
over ``[heads, chunks, 64, d]``; the chunk-to-chunk state recurrence runs in one CUDA kernel per
direction (``csrc/gdn_scan.cu``) with a reset flag at the first chunk of every document.  On CPU (and for
head dims the kernel does not cover) the recurrence is a plain loop over chunks, which is also the oracle
of the kernel.

Reference: the FLA ``chunk_gated_delta_rule`` call of the patched Gated-DeltaNet layers,
src/lmms_engine/models/qwen3_5/qwen3_5_ops.py.
"""
from __future__ import annotations

from typing import List, Tuple

import torch
import torch.nn.functional as F

from . import _cuda

CHUNK = 64

_cuda.register("b200_gdn_scan_fwd", "gdn_scan", "ppppppppp" + "iiii" + "s")
_cuda.register("b200_gdn_scan_bwd", "gdn_scan", "pppppppppppppp" + "iiii" + "s")
_cuda.register("b200_conv_silu_fwd", "gdn_conv", "pppp" + "l" + "iii" + "s")
_cuda.register("b200_conv_silu_bwd", "gdn_conv", "pppppp" + "l" + "iii" + "s")


def l2norm(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    return x * torch.rsqrt((x * x).sum(-1, keepdim=True) + eps)


def scan_ref(w, u, qt, kt, gamma, reset: List[bool]):
    """``w, qt, kt [H, n, C, dk]``, ``u [H, n, C, dv]``, ``gamma [H, n]`` -> ``(v_new, o)`` like ``u``."""
    H, n, _, dk = w.shape
    state = w.new_zeros((H, dk, u.shape[-1]))
    vs, os_ = [], []
    for i in range(n):
        if reset[i]:
            state = torch.zeros_like(state)
        v_new = u[:, i] - w[:, i] @ state
        os_.append(qt[:, i] @ state)
        vs.append(v_new)
        state = state * gamma[:, i, None, None] + kt[:, i].transpose(-1, -2) @ v_new
    return torch.stack(vs, 1), torch.stack(os_, 1)


def kernel_covers(dk: int, dv: int) -> bool:
    return dk == 128 and dv % 32 == 0


def _dense16(t: torch.Tensor) -> torch.Tensor:
    """Contiguous and 16-byte aligned (the kernels move float4s)."""
    t = t.contiguous()
    return t if t.data_ptr() % 16 == 0 else t.clone()


class _Scan(torch.autograd.Function):
    @staticmethod
    def forward(ctx, w, u, qt, kt, gamma, reset_t):
        w, u, qt, kt, gamma = (_dense16(t) for t in (w, u, qt, kt, gamma))
        H, n, _, dk = w.shape
        dv = u.shape[-1]
        vnew, o = torch.empty_like(u), torch.empty_like(u)
        hist = torch.empty((H, n, dk, dv), dtype=torch.float32, device=w.device)
        _cuda.call("b200_gdn_scan_fwd", w.data_ptr(), u.data_ptr(), qt.data_ptr(), kt.data_ptr(), gamma.data_ptr(),
                   reset_t.data_ptr(), vnew.data_ptr(), o.data_ptr(), hist.data_ptr(), H, n, dk, dv, _cuda.stream())
        ctx.save_for_backward(w, qt, kt, gamma, reset_t, vnew, hist)
        return vnew, o

    @staticmethod
    def backward(ctx, d_vnew, d_o):
        w, qt, kt, gamma, reset_t, vnew, hist = ctx.saved_tensors
        H, n, _, dk = w.shape
        dv = vnew.shape[-1]
        ns = dv // 32
        d_vnew = _dense16(d_vnew) if d_vnew is not None else torch.zeros_like(vnew)
        d_o = _dense16(d_o) if d_o is not None else torch.zeros_like(vnew)
        du = torch.empty_like(vnew)
        parts = torch.empty((3, ns, H, n, CHUNK, dk), dtype=torch.float32, device=w.device)
        dg_p = torch.empty((ns, H, n), dtype=torch.float32, device=w.device)
        _cuda.call("b200_gdn_scan_bwd", w.data_ptr(), qt.data_ptr(), kt.data_ptr(), gamma.data_ptr(), reset_t.data_ptr(),
                   vnew.data_ptr(), hist.data_ptr(), d_vnew.data_ptr(), d_o.data_ptr(), du.data_ptr(), parts[0].data_ptr(),
                   parts[1].data_ptr(), parts[2].data_ptr(), dg_p.data_ptr(), H, n, dk, dv, _cuda.stream())
        dw, dq, dk_ = parts.sum(1).unbind(0)
        return dw, du, dq, dk_, dg_p.sum(0), None


def scan(w, u, qt, kt, gamma, reset: List[bool]):
    if w.is_cuda and kernel_covers(w.shape[-1], u.shape[-1]):
        reset_t = torch.tensor([int(r) for r in reset], dtype=torch.int32, device=w.device)
        return _Scan.apply(w.float(), u.float(), qt.float(), kt.float(), gamma.float(), reset_t)
    return scan_ref(w, u, qt, kt, gamma, reset)


def chunk_plan(lengths: List[int], device) -> Tuple[torch.Tensor, torch.Tensor, List[bool]]:
    """Row maps between the packed stream and its per-document padding to whole chunks:
    ``src [Tp]`` (stream row of every padded row; ``T`` = the zero row), ``back [T]``, reset flags per chunk."""
    src, back, reset, at, T = [], [], [], 0, sum(lengths)
    for L in lengths:
        if L <= 0:
            continue
        n = (L + CHUNK - 1) // CHUNK
        base = len(src)
        src += list(range(at, at + L)) + [T] * (n * CHUNK - L)
        back += list(range(base, base + L))
        reset += [True] + [False] * (n - 1)
        at += L
    return (torch.tensor(src, dtype=torch.long, device=device), torch.tensor(back, dtype=torch.long, device=device), reset)


class _PaddedGather(torch.autograd.Function):
    """``cat([x, 0])[fwd]`` whose backward is the gather ``cat([g, 0])[bwd]`` instead of a scatter-add: every
    real row of ``x`` appears exactly once in ``fwd`` (index ``len(x)`` = the zero row) and ``bwd`` is its inverse."""

    @staticmethod
    def forward(ctx, x, fwd, bwd):
        ctx.save_for_backward(fwd, bwd)
        return torch.cat([x, x.new_zeros((1,) + x.shape[1:])], 0).index_select(0, fwd)

    @staticmethod
    def backward(ctx, g):
        fwd, bwd = ctx.saved_tensors
        return torch.cat([g, g.new_zeros((1,) + g.shape[1:])], 0).index_select(0, bwd), None, None


class _Unpad(torch.autograd.Function):
    """``x[back]`` (drop the padding rows); backward places the rows back with the gather ``cat([g, 0])[src]``."""

    @staticmethod
    def forward(ctx, x, back, src):
        ctx.save_for_backward(src)
        return x.index_select(0, back)

    @staticmethod
    def backward(ctx, g):
        (src,) = ctx.saved_tensors
        return torch.cat([g, g.new_zeros((1,) + g.shape[1:])], 0).index_select(0, src), None, None


def _unpad(x, back, src):
    return _Unpad.apply(x, back, src)


def plan_for(ctx, device):
    """``(lengths, pos_in_doc, chunk_plan)`` of a packed context: one host read of the document boundaries per
    forward pass, cached on the context and shared by all layers."""
    plan = getattr(ctx, "gdn_plan", None)
    if plan is None:
        bounds = ctx.cu_seqlens.tolist()
        lengths = [hi - lo for lo, hi in zip(bounds[:-1], bounds[1:]) if hi > lo]
        pos = torch.cat([torch.arange(n) for n in lengths]) if lengths else torch.zeros(0, dtype=torch.long)
        plan = (lengths, pos.to(device, non_blocking=True), chunk_plan(lengths, device))
        try:
            ctx.gdn_plan = plan
        except AttributeError:
            pass
    return plan


def chunk_gated_delta_rule_packed(q, k, v, g, beta, lengths: List[int], plan=None):
    """``q, k [T, H, dk]``, ``v [T, H, dv]``, ``g, beta [T, H]`` for documents of ``lengths`` laid end to end ->
    ``o [T, H, dv]``.  Math in fp32; q and k are L2-normalised here, q is scaled by ``dk ** -0.5``."""
    dt = q.dtype
    T, H, dk = k.shape
    dv = v.shape[-1]
    src, back, reset = plan if plan is not None else chunk_plan(lengths, q.device)
    n = len(reset)
    if n == 0:
        return v.new_zeros((T, H, dv))

    def lay(x):  # [T, H, ...] -> contiguous fp32 [H, n, C, ...] with zero padding rows
        # gather in the input dtype (half the bytes for bf16 streams), then one strided copy that also casts
        x = _PaddedGather.apply(x, src, back)
        x = x.view(n, CHUNK, *x.shape[1:]).movedim(2, 0)
        return torch.empty(x.shape, dtype=torch.float32, device=x.device).copy_(x)

    # padding rows are zero, so normalising after the layout change leaves them zero
    q, k = l2norm(lay(q)) * dk ** -0.5, l2norm(lay(k))
    v, g, beta = lay(v), lay(g), lay(beta)          # g, beta: [H, n, C]
    vb, kb = v * beta[..., None], k * beta[..., None]
    g = g.cumsum(-1)
    decay = (g[..., :, None] - g[..., None, :]).tril().exp().tril()
    upper = torch.triu(torch.ones(CHUNK, CHUNK, dtype=torch.bool, device=q.device))
    strict = torch.triu(torch.ones(CHUNK, CHUNK, dtype=torch.bool, device=q.device), diagonal=1)
    a = ((kb @ k.transpose(-1, -2)) * decay).masked_fill(upper, 0)
    eye = torch.eye(CHUNK, dtype=a.dtype, device=a.device)
    inv = torch.linalg.solve_triangular(eye + a, eye.expand_as(a).contiguous(), upper=False)
    u = inv @ vb                                   # values after the in-chunk corrections
    w = inv @ (kb * g.exp()[..., None])            # what the carried state contributes to them
    qt = q * g.exp()[..., None]
    kt = k * (g[..., -1:] - g).exp()[..., None]
    gamma = g[..., -1].exp()
    v_new, o_state = scan(w, u, qt, kt, gamma, reset)
    attn = ((q @ k.transpose(-1, -2)) * decay).masked_fill(strict, 0)
    out = o_state + attn @ v_new                   # [H, n, C, dv]
    # back to the stream: cast first (half the bytes for bf16 streams), one strided copy, one gather
    out = out.to(dt).movedim(0, 2).reshape(n * CHUNK, H, dv)
    # stream row t sits at padded row back[t]; the gradient of this gather is the gather by ``src`` of [g; 0]
    return _unpad(out, back, src)


def causal_conv_silu_ref(x: torch.Tensor, weight: torch.Tensor, pos_in_doc: torch.Tensor) -> torch.Tensor:
    """fp32 framework-op form (CPU path and oracle of the kernels)."""
    K = weight.shape[1]
    xf = x.float()
    acc = xf * weight[:, K - 1].float()
    for j in range(1, K):
        shifted = F.pad(xf, (0, 0, j, 0))[: xf.shape[0]]
        acc = acc + torch.where((pos_in_doc >= j).unsqueeze(1), shifted, torch.zeros_like(shifted)) * weight[:, K - 1 - j].float()
    return F.silu(acc).to(x.dtype)


class _ConvSilu(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, pos32):
        x = _dense16(x)
        w = weight.float().contiguous()
        y = torch.empty_like(x)
        _cuda.call("b200_conv_silu_fwd", x.data_ptr(), w.data_ptr(), pos32.data_ptr(), y.data_ptr(), x.shape[0], x.shape[1],
                   w.shape[1], int(x.dtype == torch.bfloat16), _cuda.stream())
        ctx.save_for_backward(x, w, pos32)
        ctx.wdtype = weight.dtype
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, pos32 = ctx.saved_tensors
        dy = _dense16(dy)
        dx = torch.empty_like(x)
        dw = torch.zeros_like(w)
        _cuda.call("b200_conv_silu_bwd", x.data_ptr(), w.data_ptr(), pos32.data_ptr(), dy.data_ptr(), dx.data_ptr(), dw.data_ptr(),
                   x.shape[0], x.shape[1], w.shape[1], int(x.dtype == torch.bfloat16), _cuda.stream())
        return dx, dw.to(ctx.wdtype), None


def causal_conv_silu_packed(x: torch.Tensor, weight: torch.Tensor, pos_in_doc: torch.Tensor) -> torch.Tensor:
    """Depthwise causal convolution inside every document followed by SiLU.  ``x [T, Ch]``,
    ``weight [Ch, K]`` (tap ``K-1`` multiplies the current token), ``pos_in_doc [T]``."""
    if (x.is_cuda and weight.shape[1] in (2, 3, 4) and x.dtype in (torch.bfloat16, torch.float32) and x.shape[0] > 0
            and x.shape[1] % 2 == 0):
        return _ConvSilu.apply(x, weight, pos_in_doc.to(torch.int32).contiguous())
    return causal_conv_silu_ref(x, weight, pos_in_doc)
