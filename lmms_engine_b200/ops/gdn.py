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


def _chunk_terms(q, k, v, g, beta, src, back, n):
    """Per-chunk quantities of the rule from packed inputs: what the scan consumes and what finishes the output."""
    dk = k.shape[-1]

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
    attn = ((q @ k.transpose(-1, -2)) * decay).masked_fill(strict, 0)
    return w, u, qt, kt, gamma, attn


def cp_plan_for(ctx, device, group):
    """Like ``plan_for`` for this rank's contiguous slice of the (padded) stream: ``(piece lengths, position of every
    local token inside its document, chunk plan, first_continues, live)``; ``live`` = local rows that are real tokens."""
    import torch.distributed as dist

    plan = getattr(ctx, "gdn_cp_plan", None)
    if plan is None:
        bounds = [int(b) for b in ctx.cu_seqlens.tolist()]
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        total = ctx.split_total or bounds[-1] + (-bounds[-1]) % world
        per = total // world
        lo, hi = rank * per, min((rank + 1) * per, bounds[-1])
        lengths, pos, first_continues = [], [], False
        for a, b in zip(bounds[:-1], bounds[1:]):
            s, e = max(a, lo), min(b, hi)
            if e > s:
                if not lengths and s > a:
                    first_continues = True
                lengths.append(e - s)
                pos.append(torch.arange(s - a, e - a))
        pos_t = torch.cat(pos) if pos else torch.zeros(0, dtype=torch.long)
        plan = (lengths, pos_t.to(device, non_blocking=True), chunk_plan(lengths, device), first_continues, max(hi - lo, 0))
        try:
            ctx.gdn_cp_plan = plan
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
    w, u, qt, kt, gamma, attn = _chunk_terms(q, k, v, g, beta, src, back, n)
    v_new, o_state = scan(w, u, qt, kt, gamma, reset)
    out = o_state + attn @ v_new                   # [H, n, C, dv]
    # back to the stream: cast first (half the bytes for bf16 streams), one strided copy, one gather
    out = out.to(dt).movedim(0, 2).reshape(n * CHUNK, H, dv)
    # stream row t sits at padded row back[t]; the gradient of this gather is the gather by ``src`` of [g; 0]
    return _unpad(out, back, src)


# ------------------------------------------------------------------------------ state hand-off between ranks
def scan_with_state(w, u, qt, kt, gamma, reset: List[bool], init=None, read_final: bool = False):
    """The chunk recurrence with a given state before the first chunk and / or the state after the last chunk read
    out, on the unchanged scan (kernel or loop).  Both are expressed as extra chunks: ``init [H, dk, dvv]`` enters
    through chunks whose keys are rows of the identity and whose values are the rows of ``init`` (no decay, no
    correction, no output), the final state leaves through chunks whose queries are rows of the identity.  Gradients
    with respect to ``init`` and of the final state follow from the scan's own backward."""
    H, n, C, dk = w.shape
    dvv = u.shape[-1]
    nf = (dk + C - 1) // C
    eye = torch.zeros((nf * C, dk), dtype=w.dtype, device=w.device)
    eye[:dk] = torch.eye(dk, dtype=w.dtype, device=w.device)
    eye = eye.view(nf, C, dk)[None].expand(H, -1, -1, -1)
    zk, zv, one = w.new_zeros((H, nf, C, dk)), u.new_zeros((H, nf, C, dvv)), gamma.new_ones((H, nf))
    reset = list(reset)
    pre = post = 0
    if init is not None:
        rows = torch.cat([init.to(u.dtype), u.new_zeros((H, nf * C - dk, dvv))], 1).view(H, nf, C, dvv)
        w, u, qt, kt, gamma = torch.cat([zk, w], 1), torch.cat([rows, u], 1), torch.cat([zk, qt], 1), torch.cat([eye, kt], 1), torch.cat([one, gamma], 1)
        reset = [True] + [False] * (nf - 1) + [False] + reset[1:]
        pre = nf
    if read_final:
        w, u, qt, kt, gamma = torch.cat([w, zk], 1), torch.cat([u, zv], 1), torch.cat([qt, eye], 1), torch.cat([kt, zk], 1), torch.cat([gamma, one], 1)
        reset = reset + [False] * nf
        post = nf
    v_new, o = scan(w.contiguous(), u.contiguous(), qt.contiguous(), kt.contiguous(), gamma.contiguous(), reset)
    final = o[:, pre + n:].reshape(H, nf * C, dvv)[:, :dk] if read_final else None
    return v_new[:, pre:pre + n], o[:, pre:pre + n], final


def chunk_gated_delta_rule_stateful(q, k, v, g, beta, state=None):
    """ONE sequence piece continued from ``state [H, dk, dv]`` (``None``: from zero): returns the outputs ``[T, H, dv]``
    and the state after the piece.  Generation uses it for the prompt and for every later token."""
    dt = q.dtype
    T, H, dk = k.shape
    src, back, reset = chunk_plan([T], q.device)
    n = len(reset)
    w, u, qt, kt, gamma, attn = _chunk_terms(q, k, v, g, beta, src, back, n)
    v_new, o_state, final = scan_with_state(w, u, qt, kt, gamma, reset, state, True)
    out = (o_state + attn @ v_new).to(dt).movedim(0, 2).reshape(n * CHUNK, H, v.shape[-1])
    return _unpad(out, back, src), final


def chunk_gated_delta_rule_cp(q, k, v, g, beta, lengths: List[int], first_continues: bool, group, plan=None):
    """The rule when the packed stream is split into contiguous token slices over the ranks of ``group`` (all heads on
    every rank).  ``lengths``: the pieces of documents inside this rank's slice; ``first_continues``: the first piece
    continues a document that began on an earlier rank.

    The state recurrence is affine in the state, so a slice acts on an incoming state ``S`` as ``A S + B``: ``B`` is the
    slice's own final state from zero, ``A`` its final state from the identity with zero values, and the outputs are
    ``out(0) + outA S``.  Every rank runs those two scans on its own slice at once (the second only when its first piece
    continues), ``A`` and ``B`` of all ranks are gathered (``[H, dk, dk]`` and ``[H, dk, dv]`` per rank) and every rank folds
    the earlier ranks' maps into its incoming state.  A document boundary inside a slice resets the state, which makes
    that slice's ``A`` zero by construction.  The reference delegates this to the FLA library's context-parallel path
    (src/lmms_engine/models/qwen3_5/qwen3_5_ops.py:183-200, 266-279)."""
    import torch.distributed as dist
    import torch.distributed.nn.functional as dist_fn

    dt = q.dtype
    T, H, dk = k.shape
    dv = v.shape[-1]
    src, back, reset = plan if plan is not None else chunk_plan(lengths, q.device)
    n = len(reset)
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    dev = q.device
    if n:
        w, u, qt, kt, gamma, attn = _chunk_terms(q, k, v, g, beta, src, back, n)
        v0, o0, B = scan_with_state(w, u, qt, kt, gamma, reset, None, True)
        out0 = o0 + attn @ v0
        if first_continues:
            ident = torch.eye(dk, dtype=torch.float32, device=dev)[None].expand(H, -1, -1)
            vA, oA, A = scan_with_state(w, torch.zeros_like(w), qt, kt, gamma, reset, ident, True)
            outA = oA + attn @ vA                     # [H, n, C, dk]: how the outputs read the incoming state
        else:
            A, outA = torch.zeros((H, dk, dk), dtype=torch.float32, device=dev), None
    else:  # an empty slice (only padding of the split) passes the state on unchanged
        B = torch.zeros((H, dk, dv), dtype=torch.float32, device=dev) + 0.0 * (q.sum() + k.sum() + v.sum() + g.sum() + beta.sum()).float()
        A = torch.eye(dk, dtype=torch.float32, device=dev)[None].expand(H, -1, -1).contiguous() if first_continues else torch.zeros((H, dk, dk), dtype=torch.float32, device=dev)
        outA = out0 = None
    packed = torch.cat([A.reshape(H, -1), B.reshape(H, -1)], 1).contiguous()
    everyone = dist_fn.all_gather(packed, group=group)
    # every rank must run the gather's backward (a collective), also the ranks that use none of its outputs
    S = torch.zeros((H, dk, dv), dtype=torch.float32, device=dev) + 0.0 * sum(e.sum() for e in everyone)
    for j in range(rank):
        Aj, Bj = everyone[j][:, : dk * dk].view(H, dk, dk), everyone[j][:, dk * dk:].view(H, dk, dv)
        S = Aj @ S + Bj
    if not n:
        return v.new_zeros((T, H, dv)) + 0.0 * S.sum().to(dt)
    out = out0 + 0.0 * S.sum() if outA is None else out0 + outA @ S[:, None]
    out = out.to(dt).movedim(0, 2).reshape(n * CHUNK, H, dv)
    return _unpad(out, back, src)


def conv_halo(x: torch.Tensor, rows: int, group):
    """The last ``rows`` rows of the previous rank's slice (zeros on the first rank), differentiably."""
    import torch.distributed as dist
    import torch.distributed.nn.functional as dist_fn

    rank = dist.get_rank(group)
    tail = x[-rows:] if x.shape[0] >= rows else torch.cat([x.new_zeros((rows - x.shape[0],) + x.shape[1:]), x], 0)
    tails = dist_fn.all_gather(tail.contiguous(), group=group)
    return tails[rank - 1] if rank > 0 else torch.zeros_like(tail) + 0.0 * tails[0]


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
