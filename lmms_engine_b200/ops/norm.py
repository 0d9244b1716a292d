"""RMSNorm / LayerNorm with optional fused residual add.

CUDA bf16 inputs run the native kernels of ``csrc/elementwise.cu``; every other input
runs the fp32 PyTorch formulation below, which is also the oracle of the GPU tests.
Semantics follow Liger's ``LigerRMSNorm(offset=0, casting_mode="llama")`` that the
reference patches in (src/lmms_engine/models/qwen2/monkey_patch.py:49-50, 110-118;
src/lmms_engine/models/qwen3_vl/monkey_patch.py:129-150).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _cuda


def rmsnorm_ref(x, w, eps: float, offset: float = 0.0, residual=None):
    xf = x.float()
    if residual is not None:
        xf = (xf + residual.float()).to(x.dtype).float()
    res_out = xf.to(x.dtype) if residual is not None else None
    rstd = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    y = (xf * rstd * (w.float() + offset)).to(x.dtype)
    return (y, res_out) if residual is not None else y


def layernorm_ref(x, w, b, eps: float):
    return torch.nn.functional.layer_norm(x.float(), (x.shape[-1],), w.float(), None if b is None else b.float(), eps).to(
        x.dtype
    )


def _native_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0


class _NormFn(torch.autograd.Function):
    """y = norm(x [+ residual]); returns (y, x + residual) when a residual is given."""

    @staticmethod
    def forward(ctx, x, residual, w, b, eps, offset, ln):
        H = x.shape[-1]
        x2 = x.reshape(-1, H).contiguous()
        r2 = residual.reshape(-1, H).contiguous() if residual is not None else None
        rows = x2.shape[0]
        y = torch.empty_like(x2)
        res_out = torch.empty_like(x2) if r2 is not None else None
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        mean = torch.empty(rows, dtype=torch.float32, device=x.device) if ln else None
        _cuda.call(
            "b200_norm_fwd", x2.data_ptr(), _cuda.ptr(r2), w.data_ptr(), _cuda.ptr(b), y.data_ptr(),
            _cuda.ptr(res_out), rstd.data_ptr(), _cuda.ptr(mean), rows, H, float(eps), float(offset), int(ln),
            _cuda.stream(),
        )
        ctx.save_for_backward(res_out if res_out is not None else x2, w, rstd, mean)
        ctx.cfg = (H, float(offset), int(ln), b is not None, residual is not None, x.shape)
        if residual is not None:
            return y.view(x.shape), res_out.view(x.shape)
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy, dres=None):
        xin, w, rstd, mean = ctx.saved_tensors
        H, offset, ln, has_b, has_res, shp = ctx.cfg
        dy2 = dy.reshape(-1, H).contiguous()
        dres2 = dres.reshape(-1, H).contiguous() if (has_res and dres is not None) else None
        rows = dy2.shape[0]
        parts = _cuda.fn("b200_num_partials")()
        dx = torch.empty_like(dy2)
        dw_part = torch.empty((parts, H), dtype=torch.float32, device=dy.device)
        db_part = torch.empty((parts, H), dtype=torch.float32, device=dy.device) if has_b else None
        dw = torch.empty(H, dtype=torch.float32, device=dy.device)
        db = torch.empty(H, dtype=torch.float32, device=dy.device) if has_b else None
        _cuda.call(
            "b200_norm_bwd", dy2.data_ptr(), xin.data_ptr(), w.data_ptr(), rstd.data_ptr(), _cuda.ptr(mean),
            _cuda.ptr(dres2), dx.data_ptr(), dw_part.data_ptr(), _cuda.ptr(db_part), dw.data_ptr(), _cuda.ptr(db),
            rows, H, offset, ln, 0, _cuda.stream(),
        )
        dxv = dx.view(shp)
        return (
            dxv,
            dxv if has_res else None,
            dw.to(w.dtype),
            db.to(w.dtype) if has_b else None,
            None,
            None,
            None,
        )


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float = 1e-6, offset: float = 0.0, residual=None):
    """RMSNorm over the last dim.  With ``residual`` returns ``(norm(x+residual), x+residual)``."""
    if _native_ok(x, w):
        return _NormFn.apply(x, residual, w, None, eps, offset, False)
    return rmsnorm_ref(x, w, eps, offset, residual)


def layernorm(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor], eps: float = 1e-6):
    if _native_ok(x, w):
        return _NormFn.apply(x, None, w, b, eps, 0.0, True)
    return layernorm_ref(x, w, b, eps)
