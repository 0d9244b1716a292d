"""Newton-Schulz orthogonalisation for Muon on the tcgen05 GEMM.

Per iteration ``A = X X^T`` (symmetric: only upper tiles computed, mirrored store),
``B = b A + c A A`` (symmetric, fused ``alpha*acc + beta*Cin`` epilogue) and
``X <- a X + B X`` (fused epilogue).  Tall matrices are never transposed: the kernel reads
``X`` MN-major to form ``X^T X`` and ``X B`` instead.  Coefficients, iteration count and
the Frobenius pre-normalisation follow the reference
(src/lmms_engine/utils/muon_utils.py:129-156), whose matmuls are one Triton kernel for
``X X^T`` (``mmt_kernel``, :28-126) plus cuBLAS.
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from . import gemm as _gemm

NS_COEFFS = (3.4445, -4.7750, 2.0315)


def newton_schulz_ref(G: torch.Tensor, steps: int = 5, eps: float = 1e-7, prenormalized: bool = False) -> torch.Tensor:
    a, b, c = NS_COEFFS
    X = G.to(torch.bfloat16) if G.is_cuda else G.float()
    tall = X.shape[0] > X.shape[1]
    if tall:
        X = X.t()
    if not prenormalized:
        X = X / (X.norm() + eps)
    for _ in range(steps):
        A = X @ X.t()
        B = b * A + c * (A @ A)
        X = a * X + B @ X
    return (X.t() if tall else X).to(G.dtype)


def newton_schulz(X: torch.Tensor, steps: int = 5, work: Optional[dict] = None, max_ctas: int = 0) -> torch.Tensor:
    """Orthogonalise a Frobenius-normalised bf16 matrix ``X [m, n]``.  Returns a bf16 tensor
    (one of two ping-pong buffers; ``X`` itself is used as one of them and is overwritten).
    ``max_ctas`` confines every product to that many SMs, so that several chains can share the GPU."""
    native = X.is_cuda and X.dtype == torch.bfloat16 and X.shape[0] % 8 == 0 and X.shape[1] % 8 == 0 and X.is_contiguous()
    if not native:
        return newton_schulz_ref(X, steps, prenormalized=True)
    a, b, c = NS_COEFFS
    m, n = X.shape
    tall = m > n
    k = n if tall else m
    if work is None:
        work = {}
    A = work.get(("A", k))
    if A is None:
        A = work[("A", k)] = torch.empty((k, k), dtype=torch.bfloat16, device=X.device)
        work[("B", k)] = torch.empty((k, k), dtype=torch.bfloat16, device=X.device)
    B = work[("B", k)]
    Y = work.get(("Y", m, n))
    if Y is None:
        Y = work[("Y", m, n)] = torch.empty_like(X)
    cur, nxt = X, Y
    for _ in range(steps):
        if tall:
            _gemm.gemm(cur, cur, a_mn_major=True, b_mn_major=True, symmetric=True, out=A, max_ctas=max_ctas)  # X^T X
        else:
            _gemm.gemm(cur, cur, symmetric=True, out=A, max_ctas=max_ctas)  # X X^T
        _gemm.gemm(A, A, alpha=c, beta=b, cin=A, symmetric=True, out=B, max_ctas=max_ctas)  # b A + c A^2
        if tall:
            _gemm.gemm(cur, B, beta=a, cin=cur, out=nxt, max_ctas=max_ctas)  # a X + X B   (B symmetric)
        else:
            _gemm.gemm(B, cur, b_mn_major=True, beta=a, cin=cur, out=nxt, max_ctas=max_ctas)  # a X + B X
        cur, nxt = nxt, cur
    return cur


GRAPH_MAX_DIM = int(os.environ.get("LMMS_B200_MUON_GRAPH_MAX_DIM", "2048"))


def newton_schulz_graphed(X: torch.Tensor, steps: int, work: dict, max_ctas: int = 0) -> torch.Tensor:
    """The same chain replayed from a CUDA graph: for small matrices the ``3 * steps`` products take a few
    microseconds each and the chain is bound by launches; one graph launch replaces them.  The graph of a shape is
    captured on first use (after one eager pass that allocates the work buffers) and owns its input and output
    buffers: the result must be consumed before the next call with the same shape on the same ``work``."""
    key = ("graph", tuple(X.shape), steps, max_ctas)
    entry = work.get(key)
    if entry is None:
        inner: dict = {}
        side = torch.cuda.Stream(device=X.device)
        side.wait_stream(torch.cuda.current_stream(X.device))
        with torch.cuda.stream(side):
            newton_schulz(X.clone(), steps, inner, max_ctas)  # allocates A / B / Y, sets kernel attributes
        torch.cuda.current_stream(X.device).wait_stream(side)
        xin, xs = torch.empty_like(X), torch.empty_like(X)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            xs.copy_(xin)  # the chain overwrites its input (ping-pong buffer)
            out = newton_schulz(xs, steps, inner, max_ctas)
        entry = work[key] = (graph, xin, out, inner)
    graph, xin, out, _ = entry
    xin.copy_(X)
    graph.replay()
    return out


def orthogonalize(X: torch.Tensor, steps: int = 5, work: Optional[dict] = None, max_ctas: int = 0) -> torch.Tensor:
    """Newton-Schulz chain, from a captured graph when the matrix is small enough to be launch-bound
    (both sides at most ``LMMS_B200_MUON_GRAPH_MAX_DIM``, default 2048; 0 turns graphs off)."""
    small = max(X.shape) <= GRAPH_MAX_DIM
    native = X.is_cuda and X.dtype == torch.bfloat16 and X.shape[0] % 8 == 0 and X.shape[1] % 8 == 0 and X.is_contiguous()
    if small and native and work is not None and not torch.cuda.is_current_stream_capturing():
        return newton_schulz_graphed(X, steps, work, max_ctas)
    return newton_schulz(X, steps, work, max_ctas)


def muon_scale(shape, rms_scale: bool = True) -> float:
    m, n = shape[0], shape[1]
    if rms_scale:
        return 0.2 * (max(m, n) ** 0.5)
    return max(1.0, m / n) ** 0.5


MUON_EXCLUDE_PATTERNS = ["emb", "norm", "lm_head", "bias", "wte", "wpe", "output", "a_proj", "b_proj", "conv1d", "rotary"]


def is_muon_param(name: str, p: torch.Tensor) -> bool:
    """2-D weights whose name matches none of the exclusion patterns
    (src/lmms_engine/train/hf/trainer.py:383-449)."""
    return p.ndim == 2 and not any(pat in name for pat in MUON_EXCLUDE_PATTERNS)


def ns_flops(shape, steps: int = 5) -> float:
    m, n = shape
    k, big = (n, m) if m > n else (m, n)
    return steps * (2.0 * k * k * big * 2 + 2.0 * k * k * k)
