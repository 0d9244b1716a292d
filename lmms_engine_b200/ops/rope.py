"""Rotary position embedding: plain, multimodal (sectioned / interleaved) and vision 2-D.

All variants reduce to a per-token ``cos/sin [T, rot_dim]`` table (built by one small
kernel from up to three position streams) followed by one apply kernel over
``[T, heads, head_dim]`` in the rotate-half convention.  Counterparts in the reference:
Liger ``liger_rotary_pos_emb`` / ``liger_multimodal_rotary_pos_emb``
(src/lmms_engine/models/qwen2/monkey_patch.py:47-48,
src/lmms_engine/models/qwen2_5_vl/monkey_patch.py:86-87) and the interleaved layout of
Qwen3-VL (src/lmms_engine/models/qwen3_vl/qwen3_vl_ops.py:502-585).
"""
from __future__ import annotations

from typing import Optional, Sequence, Tuple

import torch

from . import _cuda

MODE_PLAIN, MODE_SECTIONED, MODE_INTERLEAVED = 0, 1, 2


def inv_freq(head_dim: int, theta: float, device=None) -> torch.Tensor:
    return 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device=device) / head_dim))


def rope_table_ref(pos: torch.Tensor, invf: torch.Tensor, mode: int = 0, sections: Sequence[int] = (0, 0, 0)):
    """``pos``: [T] or [3, T] int64.  Returns fp32 ``cos, sin`` of shape [T, 2*len(invf)]."""
    if pos.dim() == 1:
        pos = pos.unsqueeze(0).expand(3, -1)
    half = invf.numel()
    ang = pos.float().unsqueeze(-1) * invf.view(1, 1, half)  # [3, T, half]
    idx = torch.arange(half, device=pos.device)
    if mode == MODE_PLAIN:
        sel = torch.zeros(half, dtype=torch.long, device=pos.device)
    elif mode == MODE_SECTIONED:
        s0, s1, _ = sections
        sel = torch.where(idx < s0, 0, torch.where(idx < s0 + s1, 1, 2))
    else:
        _, s1, s2 = sections
        m = idx % 3
        sel = torch.where((m == 1) & (idx < 3 * s1), 1, torch.where((m == 2) & (idx < 3 * s2), 2, 0))
    a = ang.gather(0, sel.view(1, 1, half).expand(1, ang.shape[1], half))[0]  # [T, half]
    a = torch.cat([a, a], dim=-1)
    return a.cos(), a.sin()


def rope_table(pos: torch.Tensor, invf: torch.Tensor, mode: int = 0, sections: Sequence[int] = (0, 0, 0)):
    if not pos.is_cuda:
        return rope_table_ref(pos, invf, mode, sections)
    if pos.dim() == 1:
        pos = pos.unsqueeze(0).expand(3, -1)
    pos = pos.contiguous().to(torch.int64)
    T = pos.shape[1]
    half = invf.numel()
    cos = torch.empty((T, 2 * half), dtype=torch.float32, device=pos.device)
    sin = torch.empty_like(cos)
    s0, s1, s2 = (int(s) for s in sections)
    _cuda.call(
        "b200_rope_table", pos.data_ptr(), invf.contiguous().data_ptr(), cos.data_ptr(), sin.data_ptr(), T, half,
        int(mode), s0, s1, s2, 1.0, _cuda.stream(),
    )
    return cos, sin


def rope_apply_ref(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, conj: bool = False) -> torch.Tensor:
    """``x``: [T, H, D]; ``cos/sin``: [T, rot_dim] with rot_dim <= D."""
    rot = cos.shape[-1]
    xr, xp = x[..., :rot].float(), x[..., rot:]
    c, s = cos.unsqueeze(1).float(), sin.unsqueeze(1).float()
    half = rot // 2
    x1, x2 = xr[..., :half], xr[..., half:]
    if not conj:
        o = torch.cat([x1 * c[..., :half] - x2 * s[..., :half], x2 * c[..., half:] + x1 * s[..., half:]], -1)
    else:
        o = torch.cat([x1 * c[..., :half] + x2 * s[..., half:], x2 * c[..., half:] - x1 * s[..., :half]], -1)
    return torch.cat([o.to(x.dtype), xp], -1)


def _apply_native(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, conj: bool, inplace: bool) -> torch.Tensor:
    T, Hn, D = x.shape
    if x.stride(2) != 1 or x.stride(1) != D:
        x = x.contiguous()
        inplace = True  # the contiguous copy is ours
    rot = cos.shape[-1]
    y = x if inplace else torch.empty((T, Hn, D), dtype=x.dtype, device=x.device)
    if rot < D and not inplace:
        y[..., rot:] = x[..., rot:]
    _cuda.call(
        "b200_rope_apply", x.data_ptr(), y.data_ptr(), cos.data_ptr(), sin.data_ptr(), T, Hn, D, rot, x.stride(0),
        y.stride(0), int(conj), _cuda.stream(),
    )
    return y


class _RopeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cos, sin):
        ctx.save_for_backward(cos, sin)
        return _apply_native(x, cos, sin, False, False)

    @staticmethod
    def backward(ctx, dy):
        cos, sin = ctx.saved_tensors
        return _apply_native(dy, cos, sin, True, False), None, None


def rope_apply(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotate ``x [T, H, D]`` by the per-token table; differentiable."""
    if x.is_cuda and x.dtype == torch.bfloat16 and cos.shape[-1] % 16 == 0 and x.shape[-1] % 8 == 0:
        if cos.dtype != torch.float32 or sin.dtype != torch.float32:
            # the kernel reads the tables as fp32; a table that some wrapper cast down would be read past its end
            raise TypeError(f"rotary tables must be float32, got {cos.dtype} / {sin.dtype}")
        if cos.shape[0] < x.shape[0]:
            raise ValueError(f"rotary table has {cos.shape[0]} rows for {x.shape[0]} tokens")
        return _RopeFn.apply(x, cos.contiguous(), sin.contiguous())
    return rope_apply_ref(x, cos, sin)


def vision_rope_table(grid_thw: torch.Tensor, head_dim: int, merge: int, theta: float = 10000.0):
    """2-D rotary table for ViT patches laid out in ``merge x merge`` blocks.

    Half of the rotary frequencies follow the patch row, half the patch column
    (upstream ``Qwen2_5_VisionTransformerPretrainedModel.rot_pos_emb``).  Returns fp32
    ``cos, sin`` of shape [sum(t*h*w), head_dim].
    """
    device = grid_thw.device
    quarter = head_dim // 4
    invf = 1.0 / (theta ** (torch.arange(0, head_dim // 2, 2, dtype=torch.float32, device=device) / (head_dim // 2)))
    pos = []
    for t, h, w in grid_thw.tolist():
        hp = torch.arange(h, device=device).unsqueeze(1).expand(h, w)
        wp = torch.arange(w, device=device).unsqueeze(0).expand(h, w)

        def blk(p):
            return p.reshape(h // merge, merge, w // merge, merge).permute(0, 2, 1, 3).reshape(-1)

        pos.append(torch.stack([blk(hp), blk(wp)], -1).repeat(t, 1))
    pos = torch.cat(pos, 0).float()  # [P, 2]
    ang = torch.cat([pos[:, :1] * invf[None, :quarter], pos[:, 1:] * invf[None, :quarter]], -1)  # [P, D/2]
    ang = torch.cat([ang, ang], -1)
    return ang.cos(), ang.sin()
