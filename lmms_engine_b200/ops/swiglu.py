"""SwiGLU: ``silu(gate) * up`` and the fused MLP built on it.

``swiglu_mlp`` runs gate and up projections in ONE tcgen05 GEMM whose epilogue applies
SiLU*mul while the accumulators are still in TMEM; gate/up pre-activations are kept
(bf16) for backward so no GEMM is recomputed.  The reference gets the elementwise part
from Liger's ``LigerSwiGLUMLP`` and the GEMMs from cuBLAS
(src/lmms_engine/models/qwen2/monkey_patch.py:76-77, 114-115).
"""
from __future__ import annotations

import torch

from . import _cuda
from . import gemm as _gemm


def swiglu_ref(g: torch.Tensor, u: torch.Tensor) -> torch.Tensor:
    return (torch.nn.functional.silu(g.float()) * u.float()).to(g.dtype)


class _SwiGLUFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, g, u):
        g = g.contiguous()
        u = u.contiguous()
        h = torch.empty_like(g)
        _cuda.call("b200_swiglu_fwd", g.data_ptr(), u.data_ptr(), h.data_ptr(), g.numel(), _cuda.stream())
        ctx.save_for_backward(g, u)
        return h

    @staticmethod
    def backward(ctx, dh):
        g, u = ctx.saved_tensors
        dh = dh.contiguous()
        dg = torch.empty_like(g)
        du = torch.empty_like(u)
        _cuda.call(
            "b200_swiglu_bwd", dh.data_ptr(), g.data_ptr(), u.data_ptr(), dg.data_ptr(), du.data_ptr(), g.numel(),
            _cuda.stream(),
        )
        return dg, du


def swiglu(g: torch.Tensor, u: torch.Tensor) -> torch.Tensor:
    if g.is_cuda and g.dtype == torch.bfloat16 and g.numel() % 8 == 0:
        return _SwiGLUFn.apply(g, u)
    return swiglu_ref(g, u)


class _SwiGLUMLPFn(torch.autograd.Function):
    """down( silu(x Wg^T) * (x Wu^T) ) with the first two GEMMs and the activation fused."""

    @staticmethod
    def forward(ctx, x, wg, wu, wd):
        shp = x.shape
        x2 = x.reshape(-1, shp[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        h, g, u = _gemm.gemm_swiglu(x2, wg, wu, store_gu=True)
        y = _gemm.matmul_nt(h, wd)
        ctx.save_for_backward(x2, wg, wu, wd, g, u)
        ctx.shp = shp
        return y.view(*shp[:-1], wd.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, wg, wu, wd, g, u = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        # recompute h (elementwise) instead of keeping a third [T, I] tensor alive
        h = torch.empty_like(g)
        _cuda.call("b200_swiglu_fwd", g.data_ptr(), u.data_ptr(), h.data_ptr(), g.numel(), _cuda.stream())
        dwd = _gemm.matmul_tn(dy2, h) if ctx.needs_input_grad[3] else None
        dh = _gemm.matmul_nn(dy2, wd, out=h)  # reuse h's storage
        # dg, du overwrite g, u in place
        _cuda.call(
            "b200_swiglu_bwd", dh.data_ptr(), g.data_ptr(), u.data_ptr(), g.data_ptr(), u.data_ptr(), g.numel(),
            _cuda.stream(),
        )
        dwg = _gemm.matmul_tn(g, x2) if ctx.needs_input_grad[1] else None
        dwu = _gemm.matmul_tn(u, x2) if ctx.needs_input_grad[2] else None
        dx = None
        if ctx.needs_input_grad[0]:
            dx = _gemm.matmul_nn(g, wg)
            dx = _gemm.gemm(u, wu, b_mn_major=True, cin=dx, beta=1.0, out=dx)
            dx = dx.view(ctx.shp)
        return dx, dwg, dwu, dwd


def swiglu_mlp(x: torch.Tensor, wg: torch.Tensor, wu: torch.Tensor, wd: torch.Tensor) -> torch.Tensor:
    native = (
        x.is_cuda
        and x.dtype == torch.bfloat16
        and wg.dtype == torch.bfloat16
        and x.shape[-1] % 8 == 0
        and wg.shape[0] % 8 == 0
        and wg.is_contiguous()
        and wu.is_contiguous()
        and wd.is_contiguous()
    )
    if native and _gemm.LINEAR_BACKEND == "tcgen05":
        return _SwiGLUMLPFn.apply(x, wg, wu, wd)
    lin = torch.nn.functional.linear
    return lin(swiglu(lin(x, wg), lin(x, wu)), wd)
