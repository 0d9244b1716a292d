"""bf16 GEMM entry points backed by the tcgen05/TMEM kernel (``csrc/gemm_sm100.cu``).

``matmul_nt / matmul_nn / matmul_tn`` cover the three products of a linear layer
(forward, input gradient, weight gradient) without materialising a transpose: the
kernel reads either operand K-major or MN-major through the UMMA descriptors.

The reference routes all of these through cuBLAS via ``nn.Linear``
(e.g. src/lmms_engine/models/qwen2/qwen2_ops.py:214-310).
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _cuda

# "tcgen05": every linear layer runs on the in-tree kernel.  "cublas": plain linears use
# the library GEMM (torch.matmul) and only the fused epilogues use the in-tree kernel.
LINEAR_BACKEND = "tcgen05"


def _ok(t: torch.Tensor) -> bool:
    return (
        t.is_cuda
        and t.dtype == torch.bfloat16
        and t.dim() == 2
        and t.stride(1) == 1
        and t.stride(0) % 8 == 0
        and t.data_ptr() % 16 == 0
    )


def gemm(
    a: torch.Tensor,
    b: torch.Tensor,
    *,
    a_mn_major: bool = False,
    b_mn_major: bool = False,
    alpha: float = 1.0,
    beta: float = 0.0,
    bias: Optional[torch.Tensor] = None,
    cin: Optional[torch.Tensor] = None,
    out: Optional[torch.Tensor] = None,
    symmetric: bool = False,
    max_ctas: int = 0,
) -> torch.Tensor:
    """``out[M,N] = alpha * opA(a) @ opB(b)^T (+ bias) (+ beta*cin)``.

    ``a`` is ``[M,K]`` (K-major) or ``[K,M]`` when ``a_mn_major``; ``b`` is ``[N,K]`` or
    ``[K,N]`` when ``b_mn_major``.  With ``symmetric`` the product must be symmetric
    (``M == N``); only the upper-triangular tiles are computed and mirrored.
    """
    if not (_ok(a) and _ok(b)):
        raise TypeError("gemm needs 2-D CUDA bf16 operands with unit inner stride, 16-byte aligned")
    if a_mn_major:
        K, M = a.shape
    else:
        M, K = a.shape
    if b_mn_major:
        Kb, N = b.shape
    else:
        N, Kb = b.shape
    if K != Kb:
        raise ValueError(f"inner dimensions differ: {K} vs {Kb}")
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
    if not _ok(out) or tuple(out.shape) != (M, N):
        raise TypeError("bad output tensor")
    if cin is not None and not _ok(cin):
        raise TypeError("bad cin tensor")
    st = _cuda.status_word(a.device)
    _cuda.call(
        "b200_gemm_bf16",
        a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, a.stride(0), b.stride(0), out.stride(0),
        int(a_mn_major), int(b_mn_major), float(alpha), float(beta), _cuda.ptr(bias), _cuda.ptr(cin),
        cin.stride(0) if cin is not None else 0, int(symmetric), int(max_ctas), st.data_ptr(), _cuda.stream(),
    )
    return out


def matmul_nt(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, out=None) -> torch.Tensor:
    """``x[M,K] @ w[N,K]^T`` (linear forward)."""
    return gemm(x, w, bias=bias, out=out)


def matmul_nn(dy: torch.Tensor, w: torch.Tensor, out=None) -> torch.Tensor:
    """``dy[M,N] @ w[N,K]`` (linear input gradient)."""
    return gemm(dy, w, b_mn_major=True, out=out)


def matmul_tn(dy: torch.Tensor, x: torch.Tensor, out=None, cin=None, beta: float = 0.0) -> torch.Tensor:
    """``dy[T,N]^T @ x[T,K]`` -> ``[N,K]`` (linear weight gradient)."""
    return gemm(dy, x, a_mn_major=True, b_mn_major=True, out=out, cin=cin, beta=beta)


def gemm_swiglu(x: torch.Tensor, wg: torch.Tensor, wu: torch.Tensor, store_gu: bool = True):
    """``h = silu(x wg^T) * (x wu^T)`` in one kernel; also returns gate/up when asked."""
    if not (_ok(x) and _ok(wg) and _ok(wu)):
        raise TypeError("gemm_swiglu needs contiguous CUDA bf16 operands")
    M, K = x.shape
    inter = wg.shape[0]
    h = torch.empty((M, inter), dtype=torch.bfloat16, device=x.device)
    g = torch.empty_like(h) if store_gu else None
    u = torch.empty_like(h) if store_gu else None
    st = _cuda.status_word(x.device)
    _cuda.call(
        "b200_gemm_swiglu_bf16",
        x.data_ptr(), wg.data_ptr(), wu.data_ptr(), h.data_ptr(), _cuda.ptr(g), _cuda.ptr(u), M, inter, K,
        x.stride(0), wg.stride(0), h.stride(0), int(store_gu), st.data_ptr(), _cuda.stream(),
    )
    return h, g, u


def gemm_stats(x: torch.Tensor, w: torch.Tensor, alpha: float = 1.0):
    """bf16 logits plus per-(row, 256-column tile) softmax partials ``(max, sum exp)``."""
    M, K = x.shape
    N = w.shape[0]
    tile_n = _cuda.fn("b200_gemm_tile_n")()
    n_tiles = (N + tile_n - 1) // tile_n
    ld = (N + 7) // 8 * 8
    logits = torch.empty((M, ld), dtype=torch.bfloat16, device=x.device)
    stats = torch.empty((M, n_tiles, 2), dtype=torch.float32, device=x.device)
    st = _cuda.status_word(x.device)
    _cuda.call(
        "b200_gemm_stats_bf16",
        x.data_ptr(), w.data_ptr(), logits.data_ptr(), stats.data_ptr(), M, N, K, x.stride(0), w.stride(0), ld,
        float(alpha), st.data_ptr(), _cuda.stream(),
    )
    return logits, stats


class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias):
        shp = x.shape
        x2 = x.reshape(-1, shp[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        ctx.save_for_backward(x2, w)
        ctx.has_bias = bias is not None
        ctx.shp = shp
        y = matmul_nt(x2, w, bias)
        return y.view(*shp[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = matmul_nn(dy2, w).view(ctx.shp)
        if ctx.needs_input_grad[1]:
            dw = matmul_tn(dy2, x2)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2.sum(0, dtype=torch.float32).to(dy2.dtype)
        return dx, dw, db


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Linear layer ``x w^T + bias``; native kernel for CUDA bf16, torch elsewhere."""
    native = (
        LINEAR_BACKEND == "tcgen05"
        and x.is_cuda
        and x.dtype == torch.bfloat16
        and w.dtype == torch.bfloat16
        and x.shape[-1] % 8 == 0
        and w.shape[0] % 8 == 0
        and w.is_contiguous()
    )
    if native:
        return _LinearFn.apply(x, w, bias)
    return torch.nn.functional.linear(x, w, bias)
