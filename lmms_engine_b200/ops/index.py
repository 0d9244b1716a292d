"""Row gather / scatter over packed token streams (unpad, pad, visual-embed scatter,
deepstack add, label gather).  Replaces ``flash_attn.bert_padding.index_first_axis`` and
``masked_scatter`` used by the reference
(src/lmms_engine/models/sequence_packing_utils.py:52-62,
src/lmms_engine/models/qwen2_5_vl/qwen2_5_vl_ops.py:157-181,
src/lmms_engine/models/qwen3_vl/qwen3_vl_ops.py:437-442).
"""
from __future__ import annotations

import torch

from . import _cuda


def _native(x: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2 and x.shape[1] % 8 == 0 and x.is_contiguous()


class _GatherFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, src, idx):
        out = torch.empty((idx.numel(), src.shape[1]), dtype=src.dtype, device=src.device)
        _cuda.call("b200_gather_rows", src.data_ptr(), idx.data_ptr(), out.data_ptr(), idx.numel(), src.shape[1], src.shape[0],
                   _cuda.status_word(src.device).data_ptr(), _cuda.stream())
        ctx.save_for_backward(idx)
        ctx.n_src = src.shape[0]
        return out

    @staticmethod
    def backward(ctx, dout):
        (idx,) = ctx.saved_tensors
        dsrc = torch.zeros((ctx.n_src, dout.shape[1]), dtype=dout.dtype, device=dout.device)
        dout = dout.contiguous()
        # indices are unique in every use of this op (a permutation or a subset)
        _cuda.call("b200_scatter_rows", dout.data_ptr(), idx.data_ptr(), dsrc.data_ptr(), idx.numel(), dout.shape[1], 0, ctx.n_src,
                   _cuda.status_word(dout.device).data_ptr(), _cuda.stream())
        return dsrc, None


def gather_rows(src: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
    """``out[i] = src[idx[i]]`` (``idx < 0`` gives a zero row).  ``idx`` must not repeat rows
    when gradients are needed."""
    if _native(src):
        return _GatherFn.apply(src, idx.to(torch.int64).contiguous())
    safe = idx.clamp(min=0)
    out = src.index_select(0, safe)
    return torch.where((idx >= 0).unsqueeze(-1), out, torch.zeros_like(out))


class _ScatterFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, base, src, idx, add):
        out = base.clone()
        _cuda.call("b200_scatter_rows", src.data_ptr(), idx.data_ptr(), out.data_ptr(), idx.numel(), src.shape[1], int(add), out.shape[0],
                   _cuda.status_word(src.device).data_ptr(), _cuda.stream())
        ctx.save_for_backward(idx)
        ctx.add = add
        return out

    @staticmethod
    def backward(ctx, dout):
        (idx,) = ctx.saved_tensors
        dout = dout.contiguous()
        dsrc = torch.empty((idx.numel(), dout.shape[1]), dtype=dout.dtype, device=dout.device)
        _cuda.call("b200_gather_rows", dout.data_ptr(), idx.data_ptr(), dsrc.data_ptr(), idx.numel(), dout.shape[1], dout.shape[0],
                   _cuda.status_word(dout.device).data_ptr(), _cuda.stream())
        if ctx.add:
            dbase = dout
        else:
            dbase = dout.clone()
            dbase.index_fill_(0, idx[idx >= 0], 0)
        return dbase, dsrc, None, None


def scatter_rows(base: torch.Tensor, src: torch.Tensor, idx: torch.Tensor, add: bool = False) -> torch.Tensor:
    """Copy of ``base`` with ``out[idx[i]] = src[i]`` (or ``+=`` when ``add``); unique ``idx``."""
    if _native(base) and _native(src):
        return _ScatterFn.apply(base, src.contiguous(), idx.to(torch.int64).contiguous(), add)
    out = base.clone()
    keep = idx >= 0
    if add:
        out.index_add_(0, idx[keep], src[keep])
    else:
        out = out.index_copy(0, idx[keep], src[keep])
    return out
