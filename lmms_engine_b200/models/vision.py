"""Vision towers on packed patches: the Qwen2.5-VL windowed ViT (RMSNorm, SwiGLU MLP,
windowed + full attention, 2x2 patch merger) and the Qwen3-VL ViT (LayerNorm, GELU MLP,
interpolated learned positions, deepstack mergers).

All images / video frames of a step form one flat ``[P, C*Tp*p*p]`` patch stream; attention
never crosses an image (``cu_seqlens`` per frame) or, in windowed layers, a window
(``cu_window_seqlens``).  It runs on the non-causal varlen tcgen05 kernel (head dims 80 and
72 are zero-padded to 128 by the TMA fill).  The patch embedding is a GEMM over flattened
patches (the reference replaces the strided Conv3d the same way,
src/lmms_engine/models/qwen3_vl/qwen3_vl_ops.py:156-173).  The towers themselves are stock
``transformers`` modules in the reference (``Qwen2_5_VisionTransformerPretrainedModel``,
``Qwen3VLVisionModel``); parameter names follow them so checkpoints load unchanged.

All index planning (window order, frame boundaries, rotary positions, bilinear position
weights) is host-side numpy over the ``grid_thw`` list, so the device never waits for it.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field, fields
from typing import Any, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import attention as attn_ops
from ..ops import gemm as gemm_ops
from ..ops import norm as norm_ops
from ..ops import rope as rope_ops
from ..ops import swiglu as swiglu_ops
from .decoder_lm import RMSNorm


@dataclass
class VisionConfig:
    model_type: str = "qwen2_5_vl"
    depth: int = 32
    hidden_size: int = 1280
    intermediate_size: int = 3420
    num_heads: int = 16
    in_channels: int = 3
    patch_size: int = 14
    temporal_patch_size: int = 2
    spatial_merge_size: int = 2
    out_hidden_size: int = 3584
    window_size: int = 112
    fullatt_block_indexes: Sequence[int] = (7, 15, 23, 31)
    tokens_per_second: int = 4
    hidden_act: str = "silu"
    # Qwen3-VL
    num_position_embeddings: int = 2304
    deepstack_visual_indexes: Sequence[int] = (8, 16, 24)
    initializer_range: float = 0.02
    extra: Dict[str, Any] = field(default_factory=dict)

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "VisionConfig":
        known = {f.name for f in fields(cls)}
        kw = {k: v for k, v in d.items() if k in known}
        kw["extra"] = {k: v for k, v in d.items() if k not in known}
        return cls(**kw)

    def to_dict(self) -> Dict[str, Any]:
        d = {f.name: getattr(self, f.name) for f in fields(self) if f.name != "extra"}
        d["fullatt_block_indexes"] = list(self.fullatt_block_indexes)
        d["deepstack_visual_indexes"] = list(self.deepstack_visual_indexes)
        d.update(self.extra)
        return d


def _grid_list(grid_thw) -> List[Tuple[int, int, int]]:
    if torch.is_tensor(grid_thw):
        grid_thw = grid_thw.tolist()
    return [(int(t), int(h), int(w)) for t, h, w in grid_thw]


def frame_cu_seqlens(grid: List[Tuple[int, int, int]]) -> np.ndarray:
    lens = np.concatenate([np.full(t, h * w, dtype=np.int64) for t, h, w in grid]) if grid else np.zeros(0, np.int64)
    return np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)


def merged_block_positions(grid, merge: int) -> np.ndarray:
    """(row, col) of every patch in stream order: patches are laid out in merge x merge blocks."""
    out = []
    for t, h, w in grid:
        r = np.arange(h).reshape(h // merge, merge, 1, 1)
        c = np.arange(w).reshape(1, 1, w // merge, merge)
        rr = np.broadcast_to(r, (h // merge, merge, w // merge, merge)).transpose(0, 2, 1, 3).reshape(-1)
        cc = np.broadcast_to(c, (h // merge, merge, w // merge, merge)).transpose(0, 2, 1, 3).reshape(-1)
        out.append(np.tile(np.stack([rr, cc], -1), (t, 1)))
    return np.concatenate(out, 0) if out else np.zeros((0, 2), np.int64)


def window_plan(grid, window_size: int, merge: int, patch: int):
    """Order of merged tokens that groups them by attention window, and the window boundaries
    in patches.  Windows are ``window_size`` pixels wide; edge windows are smaller."""
    side = window_size // merge // patch
    unit = merge * merge
    order, cu = [], [0]
    base = 0
    for t, h, w in grid:
        gh, gw = h // merge, w // merge
        idx = np.arange(t * gh * gw).reshape(t, gh, gw)
        nh, nw = -(-gh // side), -(-gw // side)
        # the upstream planner always pads by a full window when the size divides evenly; the
        # extra empty windows it creates are removed again (unique_consecutive), so skip them
        for ti in range(t):
            for a in range(nh):
                for b in range(nw):
                    blk = idx[ti, a * side:(a + 1) * side, b * side:(b + 1) * side].reshape(-1)
                    if blk.size:
                        order.append(blk + base)
                        cu.append(cu[-1] + blk.size * unit)
        base += t * gh * gw
    order = np.concatenate(order) if order else np.zeros(0, np.int64)
    return order.astype(np.int64), np.asarray(cu, dtype=np.int32)


class VisionAttention(nn.Module):
    def __init__(self, dim: int, heads: int):
        super().__init__()
        self.heads, self.head_dim = heads, dim // heads
        self.qkv = nn.Linear(dim, dim * 3, bias=True)
        self.proj = nn.Linear(dim, dim, bias=True)

    def forward(self, x, cu, cos, sin):
        P = x.shape[0]
        qkv = gemm_ops.linear(x, self.qkv.weight, self.qkv.bias).view(P, 3, self.heads, self.head_dim)
        q, k, v = qkv[:, 0], qkv[:, 1], qkv[:, 2]
        q = rope_ops.rope_apply(q, cos, sin)
        k = rope_ops.rope_apply(k, cos, sin)
        o = attn_ops.varlen_attn(q, k, v, cu, cu, causal=False, softmax_scale=1.0 / math.sqrt(self.head_dim))
        return gemm_ops.linear(o.reshape(P, -1), self.proj.weight, self.proj.bias)


class GatedVisionMLP(nn.Module):
    """SwiGLU MLP with biases (Qwen2.5-VL)."""

    def __init__(self, dim: int, inter: int):
        super().__init__()
        self.gate_proj = nn.Linear(dim, inter, bias=True)
        self.up_proj = nn.Linear(dim, inter, bias=True)
        self.down_proj = nn.Linear(inter, dim, bias=True)

    def forward(self, x):
        g = gemm_ops.linear(x, self.gate_proj.weight, self.gate_proj.bias)
        u = gemm_ops.linear(x, self.up_proj.weight, self.up_proj.bias)
        return gemm_ops.linear(swiglu_ops.swiglu(g, u), self.down_proj.weight, self.down_proj.bias)


class PlainVisionMLP(nn.Module):
    """fc1 -> activation -> fc2 (Qwen3-VL)."""

    def __init__(self, dim: int, inter: int, act: str):
        super().__init__()
        self.linear_fc1 = nn.Linear(dim, inter, bias=True)
        self.linear_fc2 = nn.Linear(inter, dim, bias=True)
        self.act = act

    def forward(self, x):
        h = gemm_ops.linear(x, self.linear_fc1.weight, self.linear_fc1.bias)
        h = F.gelu(h, approximate="tanh") if "tanh" in self.act else (F.gelu(h) if "gelu" in self.act else F.silu(h))
        return gemm_ops.linear(h, self.linear_fc2.weight, self.linear_fc2.bias)


class LayerNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.bias = nn.Parameter(torch.zeros(dim))
        self.eps = eps

    def forward(self, x):
        return norm_ops.layernorm(x, self.weight, self.bias, self.eps)


class VisionBlock(nn.Module):
    def __init__(self, cfg: VisionConfig, gated: bool):
        super().__init__()
        self.norm1 = RMSNorm(cfg.hidden_size, 1e-6) if gated else LayerNorm(cfg.hidden_size, 1e-6)
        self.norm2 = RMSNorm(cfg.hidden_size, 1e-6) if gated else LayerNorm(cfg.hidden_size, 1e-6)
        self.attn = VisionAttention(cfg.hidden_size, cfg.num_heads)
        self.mlp = (GatedVisionMLP(cfg.hidden_size, cfg.intermediate_size) if gated
                    else PlainVisionMLP(cfg.hidden_size, cfg.intermediate_size, cfg.hidden_act))

    def forward(self, x, cu, cos, sin):
        x = x + self.attn(self.norm1(x), cu, cos, sin)
        return x + self.mlp(self.norm2(x))


class PatchEmbed(nn.Module):
    """Strided Conv3d expressed as a GEMM over flattened patches; the weight keeps the conv shape."""

    def __init__(self, cfg: VisionConfig, bias: bool):
        super().__init__()
        self.proj = nn.Conv3d(cfg.in_channels, cfg.hidden_size,
                              kernel_size=(cfg.temporal_patch_size, cfg.patch_size, cfg.patch_size),
                              stride=(cfg.temporal_patch_size, cfg.patch_size, cfg.patch_size), bias=bias)

    def forward(self, patches):
        w = self.proj.weight.view(self.proj.weight.shape[0], -1)
        return gemm_ops.linear(patches.to(w.dtype), w, self.proj.bias)


class PatchMerger25(nn.Module):
    def __init__(self, out_dim: int, ctx_dim: int, merge: int):
        super().__init__()
        self.hidden = ctx_dim * merge * merge
        self.ln_q = RMSNorm(ctx_dim, 1e-6)
        self.mlp = nn.Sequential(nn.Linear(self.hidden, self.hidden), nn.GELU(), nn.Linear(self.hidden, out_dim))

    def forward(self, x):
        x = self.ln_q(x).view(-1, self.hidden)
        x = F.gelu(gemm_ops.linear(x, self.mlp[0].weight, self.mlp[0].bias))
        return gemm_ops.linear(x, self.mlp[2].weight, self.mlp[2].bias)


class PatchMerger3(nn.Module):
    def __init__(self, cfg: VisionConfig, postshuffle: bool):
        super().__init__()
        self.hidden = cfg.hidden_size * cfg.spatial_merge_size ** 2
        self.postshuffle = postshuffle
        self.norm = LayerNorm(self.hidden if postshuffle else cfg.hidden_size, 1e-6)
        self.linear_fc1 = nn.Linear(self.hidden, self.hidden)
        self.linear_fc2 = nn.Linear(self.hidden, cfg.out_hidden_size)

    def forward(self, x):
        x = self.norm(x.view(-1, self.hidden)) if self.postshuffle else self.norm(x).view(-1, self.hidden)
        x = F.gelu(gemm_ops.linear(x, self.linear_fc1.weight, self.linear_fc1.bias))
        return gemm_ops.linear(x, self.linear_fc2.weight, self.linear_fc2.bias)


class _TowerBase(nn.Module):
    def _rotary(self, grid, device, order_units: Optional[np.ndarray] = None):
        cfg = self.cfg
        hd = cfg.hidden_size // cfg.num_heads
        pos = merged_block_positions(grid, cfg.spatial_merge_size)
        if order_units is not None:
            unit = cfg.spatial_merge_size ** 2
            pos = pos.reshape(-1, unit, 2)[order_units].reshape(-1, 2)
        quarter = hd // 4
        invf = 1.0 / (10000.0 ** (np.arange(0, hd // 2, 2, dtype=np.float64) / (hd // 2)))
        ang = np.concatenate([pos[:, :1] * invf[None, :quarter], pos[:, 1:] * invf[None, :quarter]], -1)
        ang = np.concatenate([ang, ang], -1).astype(np.float32)
        t = torch.from_numpy(ang).to(device, non_blocking=True)
        return t.cos(), t.sin()

    def _init_weights(self, m):
        std = self.cfg.initializer_range
        if isinstance(m, (nn.Linear, nn.Conv3d)):
            nn.init.normal_(m.weight, 0.0, std)
            if m.bias is not None:
                nn.init.zeros_(m.bias)
        elif isinstance(m, nn.Embedding):
            nn.init.normal_(m.weight, 0.0, std)


class Qwen25VisionTower(_TowerBase):
    def __init__(self, cfg: VisionConfig):
        super().__init__()
        self.cfg = cfg
        self.patch_embed = PatchEmbed(cfg, bias=False)
        self.blocks = nn.ModuleList([VisionBlock(cfg, gated=True) for _ in range(cfg.depth)])
        self.merger = PatchMerger25(cfg.out_hidden_size, cfg.hidden_size, cfg.spatial_merge_size)
        self.gradient_checkpointing = False
        self.apply(self._init_weights)

    def forward(self, patches: torch.Tensor, grid_thw) -> torch.Tensor:
        cfg = self.cfg
        grid = _grid_list(grid_thw)
        dev = patches.device
        unit = cfg.spatial_merge_size ** 2
        order, cu_win = window_plan(grid, cfg.window_size, cfg.spatial_merge_size, cfg.patch_size)
        cu_full = torch.from_numpy(frame_cu_seqlens(grid)).to(dev, non_blocking=True)
        cu_win_t = torch.from_numpy(cu_win).to(dev, non_blocking=True)
        order_t = torch.from_numpy(order).to(dev, non_blocking=True)
        cos, sin = self._rotary(grid, dev, order)
        x = self.patch_embed(patches)
        P = x.shape[0]
        x = x.view(P // unit, unit, -1).index_select(0, order_t).reshape(P, -1)
        full = set(cfg.fullatt_block_indexes)
        for i, blk in enumerate(self.blocks):
            cu = cu_full if i in full else cu_win_t
            if self.gradient_checkpointing and self.training:
                x = torch.utils.checkpoint.checkpoint(blk, x, cu, cos, sin, use_reentrant=False)
            else:
                x = blk(x, cu, cos, sin)
        merged = self.merger(x)
        inverse = torch.from_numpy(np.argsort(order)).to(dev, non_blocking=True)
        return merged.index_select(0, inverse)


class Qwen3VisionTower(_TowerBase):
    def __init__(self, cfg: VisionConfig):
        super().__init__()
        self.cfg = cfg
        self.patch_embed = PatchEmbed(cfg, bias=True)
        self.pos_embed = nn.Embedding(cfg.num_position_embeddings, cfg.hidden_size)
        self.side = int(cfg.num_position_embeddings ** 0.5)
        self.blocks = nn.ModuleList([VisionBlock(cfg, gated=False) for _ in range(cfg.depth)])
        self.merger = PatchMerger3(cfg, postshuffle=False)
        self.deepstack_merger_list = nn.ModuleList([PatchMerger3(cfg, postshuffle=True) for _ in cfg.deepstack_visual_indexes])
        self.gradient_checkpointing = False
        self.apply(self._init_weights)

    def _interp_plan(self, grid):
        """Bilinear taps into the side x side learned table for every patch, in stream order."""
        m = self.cfg.spatial_merge_size
        idx4, w4 = [[], [], [], []], [[], [], [], []]
        for t, h, w in grid:
            hs = np.linspace(0, self.side - 1, h)
            ws = np.linspace(0, self.side - 1, w)
            h0, w0 = hs.astype(np.int64), ws.astype(np.int64)
            h1, w1 = np.minimum(h0 + 1, self.side - 1), np.minimum(w0 + 1, self.side - 1)
            dh, dw = hs - h0, ws - w0
            taps = [(h0, w0, (1 - dh)[:, None] * (1 - dw)[None]), (h0, w1, (1 - dh)[:, None] * dw[None]),
                    (h1, w0, dh[:, None] * (1 - dw)[None]), (h1, w1, dh[:, None] * dw[None])]
            for i, (hh, ww, wt) in enumerate(taps):
                ind = (hh[:, None] * self.side + ww[None])
                # stream order: merge x merge blocks, repeated over frames
                blk = lambda a: np.tile(a.reshape(h // m, m, w // m, m).transpose(0, 2, 1, 3).reshape(-1), t)
                idx4[i].append(blk(ind))
                w4[i].append(blk(wt))
        return (np.stack([np.concatenate(a) for a in idx4]), np.stack([np.concatenate(a) for a in w4]).astype(np.float32))

    def forward(self, patches: torch.Tensor, grid_thw):
        cfg = self.cfg
        grid = _grid_list(grid_thw)
        dev = patches.device
        x = self.patch_embed(patches)
        idx, wt = self._interp_plan(grid)
        idx_t = torch.from_numpy(idx).to(dev, non_blocking=True)
        wt_t = torch.from_numpy(wt).to(dev, non_blocking=True).to(x.dtype)
        pos = (self.pos_embed(idx_t) * wt_t.unsqueeze(-1)).sum(0)
        x = x + pos.to(x.dtype)
        cu = torch.from_numpy(frame_cu_seqlens(grid)).to(dev, non_blocking=True)
        cos, sin = self._rotary(grid, dev)
        deep = []
        taps = list(cfg.deepstack_visual_indexes)
        for i, blk in enumerate(self.blocks):
            if self.gradient_checkpointing and self.training:
                x = torch.utils.checkpoint.checkpoint(blk, x, cu, cos, sin, use_reentrant=False)
            else:
                x = blk(x, cu, cos, sin)
            if i in taps:
                deep.append(self.deepstack_merger_list[taps.index(i)](x))
        return self.merger(x), deep
