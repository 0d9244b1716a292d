"""Fused linear + cross-entropy: the ``[T, V]`` fp32 logits are never materialised.

Per chunk of rows the tcgen05 GEMM writes bf16 logits and, from its epilogue, per-tile
softmax partials; a small kernel turns them into ``lse`` and per-row losses; for
``mean``/``sum`` reductions the gradient of the logits is formed in place right away and
fed to the two gradient GEMMs, so backward is a scale.  ``none`` keeps per-row losses
differentiable (needed by the sequence-parallel loss gather) and recomputes the logits
chunk in backward.

Reference counterpart: Liger ``LigerFusedLinearCrossEntropyLoss`` as called from
src/lmms_engine/models/qwen2/qwen2_liger.py:138-143 and
src/lmms_engine/models/common_ops/loss.py:99-103.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F

from . import _cuda
from . import gemm as _gemm

IGNORE_INDEX = -100
DEFAULT_CHUNK_ROWS = 8192


def flce_ref(hidden, weight, labels, reduction="mean", ignore_index=IGNORE_INDEX, bias=None):
    logits = F.linear(hidden, weight, bias).float()
    return F.cross_entropy(logits, labels, ignore_index=ignore_index, reduction=reduction)


def _chunk_forward(h_c, weight, labels_c, ignore_index):
    logits, stats = _gemm.gemm_stats(h_c, weight)
    rows = h_c.shape[0]
    lse = torch.empty(rows, dtype=torch.float32, device=h_c.device)
    loss = torch.empty(rows, dtype=torch.float32, device=h_c.device)
    _cuda.call(
        "b200_ce_finalize", stats.data_ptr(), logits.data_ptr(), labels_c.data_ptr(), lse.data_ptr(),
        loss.data_ptr(), rows, stats.shape[1], logits.stride(0), weight.shape[0], ignore_index, _cuda.stream(),
    )
    return logits, lse, loss


def _dlogits_(logits, lse, labels_c, gscale, V, ignore_index):
    _cuda.call(
        "b200_ce_dlogits", logits.data_ptr(), lse.data_ptr(), labels_c.data_ptr(), gscale.data_ptr(),
        logits.shape[0], logits.stride(0), V, ignore_index, _cuda.stream(),
    )


class _FLCEReduced(torch.autograd.Function):
    """mean / sum reduction; gradients are produced during forward."""

    @staticmethod
    def forward(ctx, hidden, weight, labels, mean, ignore_index, chunk_rows):
        T, H = hidden.shape
        V = weight.shape[0]
        labels = labels.contiguous().to(torch.int64)
        n_valid = (labels != ignore_index).sum().to(torch.float32)
        gscale = (1.0 / n_valid.clamp(min=1.0)).reshape(1) if mean else torch.ones(1, dtype=torch.float32, device=hidden.device)
        need_dh = ctx.needs_input_grad[0]
        need_dw = ctx.needs_input_grad[1]
        dH = torch.empty_like(hidden) if need_dh else None
        dW = torch.empty_like(weight) if need_dw else None
        total = torch.zeros((), dtype=torch.float32, device=hidden.device)
        first = True
        for r0 in range(0, T, chunk_rows):
            r1 = min(T, r0 + chunk_rows)
            h_c = hidden[r0:r1]
            lab_c = labels[r0:r1]
            logits, lse, loss = _chunk_forward(h_c, weight, lab_c, ignore_index)
            total = total + loss.sum()
            if need_dh or need_dw:
                _dlogits_(logits, lse, lab_c, gscale, V, ignore_index)
                dl = logits[:, :V]
                if need_dh:
                    _gemm.matmul_nn(dl, weight, out=dH[r0:r1])
                if need_dw:
                    if first:
                        _gemm.matmul_tn(dl, h_c, out=dW)
                    else:
                        _gemm.matmul_tn(dl, h_c, out=dW, cin=dW, beta=1.0)
                first = False
            del logits
        ctx.save_for_backward(dH, dW)
        return total * gscale[0] if mean else total

    @staticmethod
    def backward(ctx, g):
        dH, dW = ctx.saved_tensors
        # g is the upstream scalar (1 for a plain loss.backward(); 1/accum under accumulation)
        if dH is not None:
            dH = dH * g.to(dH.dtype)
        if dW is not None:
            dW = dW * g.to(dW.dtype)
        return dH, dW, None, None, None, None


class _FLCENone(torch.autograd.Function):
    """Per-row losses; the logits chunk is recomputed in backward."""

    @staticmethod
    def forward(ctx, hidden, weight, labels, ignore_index, chunk_rows):
        T = hidden.shape[0]
        labels = labels.contiguous().to(torch.int64)
        losses, lses = [], []
        for r0 in range(0, T, chunk_rows):
            r1 = min(T, r0 + chunk_rows)
            logits, lse, loss = _chunk_forward(hidden[r0:r1], weight, labels[r0:r1], ignore_index)
            losses.append(loss)
            lses.append(lse)
            del logits
        ctx.save_for_backward(hidden, weight, labels)
        ctx.cfg = (ignore_index, chunk_rows)
        return torch.cat(losses) if len(losses) > 1 else losses[0]

    @staticmethod
    def backward(ctx, g_rows):
        hidden, weight, labels = ctx.saved_tensors
        ignore_index, chunk_rows = ctx.cfg
        T, V = hidden.shape[0], weight.shape[0]
        one = torch.ones(1, dtype=torch.float32, device=hidden.device)
        dH = torch.empty_like(hidden) if ctx.needs_input_grad[0] else None
        dW = torch.empty_like(weight) if ctx.needs_input_grad[1] else None
        first = True
        for r0 in range(0, T, chunk_rows):
            r1 = min(T, r0 + chunk_rows)
            h_c, lab_c = hidden[r0:r1], labels[r0:r1]
            logits, lse, _ = _chunk_forward(h_c, weight, lab_c, ignore_index)
            _dlogits_(logits, lse, lab_c, one, V, ignore_index)
            dl = logits[:, :V]
            dl.mul_(g_rows[r0:r1].to(dl.dtype).unsqueeze(1))
            if dH is not None:
                _gemm.matmul_nn(dl, weight, out=dH[r0:r1])
            if dW is not None:
                if first:
                    _gemm.matmul_tn(dl, h_c, out=dW)
                else:
                    _gemm.matmul_tn(dl, h_c, out=dW, cin=dW, beta=1.0)
            first = False
        return dH, dW, None, None, None


def fused_linear_cross_entropy(
    hidden: torch.Tensor,
    weight: torch.Tensor,
    labels: torch.Tensor,
    reduction: str = "mean",
    ignore_index: int = IGNORE_INDEX,
    chunk_rows: int = DEFAULT_CHUNK_ROWS,
) -> torch.Tensor:
    """Cross-entropy of ``hidden @ weight.T`` against ``labels`` (already shifted)."""
    if reduction not in ("mean", "sum", "none"):
        raise ValueError(reduction)
    native = (
        hidden.is_cuda
        and hidden.dtype == torch.bfloat16
        and weight.dtype == torch.bfloat16
        and hidden.dim() == 2
        and hidden.shape[1] % 8 == 0
        and weight.shape[0] % 8 == 0
        and weight.is_contiguous()
    )
    if not native:
        return flce_ref(hidden, weight, labels, reduction, ignore_index)
    hidden = hidden.contiguous()
    if reduction == "none":
        return _FLCENone.apply(hidden, weight, labels, ignore_index, chunk_rows)
    return _FLCEReduced.apply(hidden, weight, labels, reduction == "mean", ignore_index, chunk_rows)
