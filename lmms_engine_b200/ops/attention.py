"""Packed variable-length attention.

``varlen_attn`` keeps the signature of the reference dispatcher
(src/lmms_engine/kernels/attention.py:20-51): flat ``q [Tq, Hq, D]``, ``k/v [Tk, Hkv, D]``
plus ``cu_seqlens`` boundaries, causal or full, optional left sliding window, GQA.
CUDA bf16 inputs run the tcgen05 kernels of ``csrc/attention_sm100.cu``; anything else
runs a per-document fp32 reference (also the oracle of the GPU tests).
"""
from __future__ import annotations

import math
import os
from typing import Optional, Tuple

import torch

from . import _cuda

_cuda.register("b200_attn_fwd", "attention_sm100", "ppppppp" + "iiiiii" + "llll" + "fii" + "ps")
_cuda.register("b200_attn_bwd", "attention_sm100", "ppppppppppppp" + "iiiiii" + "llllllll" + "fii" + "ps")
_cuda.register("b200_attn_bwd_v2", "attention_bwd_sm100", "pppppppppppp" + "iiiiii" + "llllllll" + "fii" + "ps")

# "split": dK/dV and dQ in two reduction-free kernels (default); "fused": the single-kernel
# variant that reduces dQ across key blocks with fp32 red.global
BACKWARD_IMPL = os.environ.get("LMMS_B200_ATTN_BWD", "split")


def varlen_attn_ref(q, k, v, cu_q, cu_k, causal=True, softmax_scale=None, window_left: int = -1):
    """fp32 per-document attention; bottom-right aligned causal mask like flash-attn."""
    Hq, Hkv, D = q.shape[1], k.shape[1], q.shape[2]
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(D)
    out = torch.empty_like(q)
    cq, ck = cu_q.tolist(), cu_k.tolist()
    for d in range(len(cq) - 1):
        qd = q[cq[d] : cq[d + 1]].float().transpose(0, 1)  # [Hq, Lq, D]
        kd = k[ck[d] : ck[d + 1]].float().transpose(0, 1)
        vd = v[ck[d] : ck[d + 1]].float().transpose(0, 1)
        if Hq != Hkv:
            kd = kd.repeat_interleave(Hq // Hkv, 0)
            vd = vd.repeat_interleave(Hq // Hkv, 0)
        lq, lk = qd.shape[1], kd.shape[1]
        s = torch.matmul(qd, kd.transpose(1, 2)) * scale
        qi = torch.arange(lq, device=q.device).unsqueeze(1) + (lk - lq)
        kj = torch.arange(lk, device=q.device).unsqueeze(0)
        mask = torch.ones(lq, lk, dtype=torch.bool, device=q.device)
        if causal:
            mask &= kj <= qi
        if window_left >= 0:
            mask &= kj >= qi - window_left
        s = s.masked_fill(~mask, float("-inf"))
        p = torch.softmax(s, dim=-1)
        p = torch.nan_to_num(p, nan=0.0)
        out[cq[d] : cq[d + 1]] = torch.matmul(p, vd).transpose(0, 1).to(q.dtype)
    return out


def _token_stride_ok(t: torch.Tensor) -> bool:
    return t.stride(2) == 1 and t.stride(1) == t.shape[2] and t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0


class _VarlenAttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, cu_q, cu_k, causal, scale, window_left):
        q = q if _token_stride_ok(q) else q.contiguous()
        k = k if _token_stride_ok(k) else k.contiguous()
        v = v if _token_stride_ok(v) else v.contiguous()
        Tq, Hq, D = q.shape
        Tk, Hkv, _ = k.shape
        o = torch.empty((Tq, Hq, D), dtype=q.dtype, device=q.device)
        lse = torch.empty((Hq, Tq), dtype=torch.float32, device=q.device)
        st = _cuda.status_word(q.device)
        _cuda.call(
            "b200_attn_fwd", q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(), cu_q.data_ptr(),
            cu_k.data_ptr(), cu_q.numel() - 1, Tq, Tk, Hq, Hkv, D, q.stride(0), k.stride(0), v.stride(0), o.stride(0),
            float(scale), int(causal), int(window_left), st.data_ptr(), _cuda.stream(),
        )
        ctx.save_for_backward(q, k, v, o, lse, cu_q, cu_k)
        ctx.cfg = (causal, scale, window_left)
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse, cu_q, cu_k = ctx.saved_tensors
        causal, scale, window_left = ctx.cfg
        do = do if _token_stride_ok(do) else do.contiguous()
        Tq, Hq, D = q.shape
        Tk, Hkv, _ = k.shape
        dq = torch.empty((Tq, Hq, D), dtype=q.dtype, device=q.device)
        dk = torch.empty((Tk, Hkv, D), dtype=q.dtype, device=q.device)
        dv = torch.empty((Tk, Hkv, D), dtype=q.dtype, device=q.device)
        delta = torch.empty((Hq, Tq), dtype=torch.float32, device=q.device)
        st = _cuda.status_word(q.device)
        if BACKWARD_IMPL == "split":
            # two reduction-free kernels (dK/dV per key block, dQ per query block)
            _cuda.call(
                "b200_attn_bwd_v2", q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), do.data_ptr(),
                lse.data_ptr(), delta.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), cu_q.data_ptr(),
                cu_k.data_ptr(), cu_q.numel() - 1, Tq, Tk, Hq, Hkv, D, q.stride(0), k.stride(0), v.stride(0),
                o.stride(0), do.stride(0), dq.stride(0), dk.stride(0), dv.stride(0), float(scale), int(causal),
                int(window_left), st.data_ptr(), _cuda.stream(),
            )
            return dq, dk, dv, None, None, None, None, None
        dq_acc = torch.empty((Tq, Hq, D), dtype=torch.float32, device=q.device)
        _cuda.call(
            "b200_attn_bwd", q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), do.data_ptr(), lse.data_ptr(),
            delta.data_ptr(), dq_acc.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), cu_q.data_ptr(),
            cu_k.data_ptr(), cu_q.numel() - 1, Tq, Tk, Hq, Hkv, D, q.stride(0), k.stride(0), v.stride(0), o.stride(0),
            do.stride(0), dq.stride(0), dk.stride(0), dv.stride(0), float(scale), int(causal), int(window_left),
            st.data_ptr(), _cuda.stream(),
        )
        return dq, dk, dv, None, None, None, None, None


def varlen_attn(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    cu_seqlens_q: torch.Tensor,
    cu_seqlens_k: Optional[torch.Tensor] = None,
    max_seqlen_q: Optional[int] = None,
    max_seqlen_k: Optional[int] = None,
    causal: bool = True,
    softmax_scale: Optional[float] = None,
    window_size: Tuple[int, int] = (-1, -1),
    dropout_p: float = 0.0,
    backend: Optional[str] = None,
) -> torch.Tensor:
    """Attention over packed documents.  ``max_seqlen_*`` are accepted for signature
    compatibility; the kernel derives its schedule from ``cu_seqlens`` on the device, so
    no host synchronisation is needed to obtain them."""
    if dropout_p != 0.0:
        raise NotImplementedError("attention dropout is not supported")
    if cu_seqlens_k is None:
        cu_seqlens_k = cu_seqlens_q
    D = q.shape[-1]
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(D)
    window_left = int(window_size[0]) if window_size is not None else -1
    window_right = int(window_size[1]) if window_size is not None and len(window_size) > 1 else -1
    if window_right >= 0 and not causal:
        # a causal mask already limits the right side to 0; a finite right window without it is a
        # different mask, which neither the kernel nor the reference formulation below implements
        raise NotImplementedError(f"window_size[1] = {window_right} (right window) is only supported together with causal=True")
    native = q.is_cuda and q.dtype == torch.bfloat16 and D % 8 == 0 and D <= 128 and backend != "reference"
    if native:
        cu_q = cu_seqlens_q.to(torch.int32).contiguous()
        cu_k = cu_seqlens_k.to(torch.int32).contiguous()
        return _VarlenAttnFn.apply(q, k, v, cu_q, cu_k, bool(causal), float(scale), window_left)
    return varlen_attn_ref(q, k, v, cu_seqlens_q, cu_seqlens_k, causal, scale, window_left)
