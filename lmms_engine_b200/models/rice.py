"""Rice vision tower of LLaVA-OneVision-1.5: a Qwen2-VL style packed ViT (LayerNorm blocks, fused
qkv, 2-D rotary positions in merged-block order) with one class token in front of every frame, a
learned rotary angle for that token, a pre-LayerNorm, and a LayerNorm + two-layer GELU merger over
2x2 patch blocks.

Behaviour follows src/lmms_engine/models/llava_onevision1_5/modeling_llavaonevision1_5.py:236-296
(rotary, patch embedding, merger), :439-465 (block) and :925-1100 (tower forward); parameter names
are the upstream ones so hub checkpoints load under ``model.visual.*``.  The class tokens are placed
with one gather instead of the per-frame copy loop, and every frame's patch rows are read back from
its own span of the class-token layout.
"""
from __future__ import annotations

import math

import numpy as np
import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import attention as attn_ops
from ..ops import gemm as gemm_ops
from ..ops import rope as rope_ops
from .vision import LayerNorm, VisionConfig, _grid_list, merged_block_positions


def _act(h, name: str):
    if "tanh" in name:
        return F.gelu(h, approximate="tanh")
    if name == "quick_gelu":
        return h * torch.sigmoid(1.702 * h)
    return F.gelu(h) if "gelu" in name else F.silu(h)


class RiceMLP(nn.Module):
    def __init__(self, dim: int, inter: int, act: str):
        super().__init__()
        self.fc1 = nn.Linear(dim, inter)
        self.fc2 = nn.Linear(inter, dim)
        self.act = act

    def forward(self, x):
        return gemm_ops.linear(_act(gemm_ops.linear(x, self.fc1.weight, self.fc1.bias), self.act), self.fc2.weight, self.fc2.bias)


def _rotate(x, cos, sin):
    """Half-split rotation in fp32 with autograd through ``cos`` / ``sin`` (class-token rows only)."""
    xf = x.float()
    h = xf.shape[-1] // 2
    rot = torch.cat([-xf[..., h:], xf[..., :h]], -1)
    return (xf * cos.unsqueeze(1) + rot * sin.unsqueeze(1)).to(x.dtype)


class RiceAttention(nn.Module):
    def __init__(self, dim: int, heads: int):
        super().__init__()
        self.heads, self.head_dim = heads, dim // heads
        self.qkv = nn.Linear(dim, dim * 3, bias=True)
        self.proj = nn.Linear(dim, dim)

    def forward(self, x, cu, cos, sin, cls_rows, cls_cos, cls_sin):
        P = x.shape[0]
        qkv = gemm_ops.linear(x, self.qkv.weight, self.qkv.bias).view(P, 3, self.heads, self.head_dim)
        q, k, v = qkv[:, 0], qkv[:, 1], qkv[:, 2]
        qr = rope_ops.rope_apply(q, cos, sin)
        kr = rope_ops.rope_apply(k, cos, sin)
        if cls_cos.requires_grad:
            # the class token's angle is a parameter: its few rows are rotated under autograd
            qr = qr.index_copy(0, cls_rows, _rotate(q.index_select(0, cls_rows), cls_cos, cls_sin))
            kr = kr.index_copy(0, cls_rows, _rotate(k.index_select(0, cls_rows), cls_cos, cls_sin))
        o = attn_ops.varlen_attn(qr, kr, v, cu, cu, causal=False, softmax_scale=1.0 / math.sqrt(self.head_dim))
        return gemm_ops.linear(o.reshape(P, -1), self.proj.weight, self.proj.bias)


class RiceBlock(nn.Module):
    def __init__(self, cfg: VisionConfig):
        super().__init__()
        self.norm1 = LayerNorm(cfg.hidden_size, 1e-5)
        self.norm2 = LayerNorm(cfg.hidden_size, 1e-5)
        self.attn = RiceAttention(cfg.hidden_size, cfg.num_heads)
        self.mlp = RiceMLP(cfg.hidden_size, cfg.intermediate_size, cfg.hidden_act)

    def forward(self, x, cu, cos, sin, cls_rows, cls_cos, cls_sin):
        x = x + self.attn(self.norm1(x), cu, cos, sin, cls_rows, cls_cos, cls_sin)
        return x + self.mlp(self.norm2(x))


class RicePatchEmbed(nn.Module):
    """Strided Conv2d over single-frame patches as a GEMM; the weight keeps the convolution's shape."""

    def __init__(self, cfg: VisionConfig):
        super().__init__()
        self.proj = nn.Conv2d(cfg.in_channels, cfg.hidden_size, kernel_size=cfg.patch_size, stride=cfg.patch_size, bias=False)

    def forward(self, patches):
        w = self.proj.weight.view(self.proj.weight.shape[0], -1)
        return gemm_ops.linear(patches.reshape(-1, w.shape[1]).to(w.dtype), w, None)


class RiceMerger(nn.Module):
    def __init__(self, out_dim: int, ctx_dim: int, merge: int, eps: float):
        super().__init__()
        self.hidden = ctx_dim * merge * merge
        self.ln_q = LayerNorm(ctx_dim, eps)
        self.mlp = nn.Sequential(nn.Linear(self.hidden, self.hidden), nn.GELU(), nn.Linear(self.hidden, out_dim))

    def forward(self, x):
        x = self.ln_q(x).view(-1, self.hidden)
        x = F.gelu(gemm_ops.linear(x, self.mlp[0].weight, self.mlp[0].bias))
        return gemm_ops.linear(x, self.mlp[2].weight, self.mlp[2].bias)


class RiceVisionTower(nn.Module):
    def __init__(self, cfg: VisionConfig):
        super().__init__()
        self.cfg = cfg
        hd = cfg.hidden_size // cfg.num_heads
        eps = float(cfg.extra.get("layer_norm_eps", 1e-5))
        self.patch_embed = RicePatchEmbed(cfg)
        self.class_embedding = nn.Parameter(cfg.hidden_size ** -0.5 * torch.randn(cfg.hidden_size))
        self.class_pos_emb = nn.Parameter(torch.randn(1, hd // 2))
        self.pre_layernorm = LayerNorm(cfg.hidden_size, eps)
        self.blocks = nn.ModuleList([RiceBlock(cfg) for _ in range(cfg.depth)])
        self.merger = RiceMerger(cfg.out_hidden_size, cfg.hidden_size, cfg.spatial_merge_size, eps)
        self.gradient_checkpointing = False
        std = cfg.initializer_range
        for m in self.modules():
            if isinstance(m, (nn.Linear, nn.Conv2d)):
                nn.init.normal_(m.weight, 0.0, std)
                if m.bias is not None:
                    nn.init.zeros_(m.bias)

    def _plan(self, grid):
        """Row maps between the patch layout and the layout with one class token per frame."""
        frames = [h * w for t, h, w in grid for _ in range(t)]
        src, cu, cls_rows, keep = [], [0], [], []
        at = 0
        for n in frames:
            cls_rows.append(len(src))
            src.append(-1)
            first = len(src)
            src.extend(range(at, at + n))
            keep.extend(range(first, first + n))
            at += n
            cu.append(len(src))
        return (np.asarray(src, np.int64), np.asarray(cu, np.int32), np.asarray(cls_rows, np.int64), np.asarray(keep, np.int64))

    def forward(self, patches: torch.Tensor, grid_thw) -> torch.Tensor:
        cfg = self.cfg
        grid = _grid_list(grid_thw)
        dev = patches.device
        hd = cfg.hidden_size // cfg.num_heads
        src, cu, cls_rows, keep = (torch.from_numpy(a).to(dev, non_blocking=True) for a in self._plan(grid))
        x = self.patch_embed(patches)
        is_cls = (src < 0).unsqueeze(-1)
        x = torch.where(is_cls, self.class_embedding.to(x.dtype).unsqueeze(0), x.index_select(0, src.clamp(min=0)))
        # rotary angles: (row, column) of every patch on hd/4 frequencies each; the class token's are learned
        pos = merged_block_positions(grid, cfg.spatial_merge_size)
        invf = 1.0 / (10000.0 ** (np.arange(0, hd // 2, 2, dtype=np.float64) / (hd // 2)))
        ang = np.concatenate([pos[:, :1] * invf[None], pos[:, 1:] * invf[None]], -1).astype(np.float32)
        ang = torch.from_numpy(ang).to(dev, non_blocking=True)
        cls_ang = self.class_pos_emb.float()
        full = torch.where(is_cls, cls_ang.detach(), ang.index_select(0, src.clamp(min=0)))
        full = torch.cat([full, full], -1)
        cos, sin = full.cos(), full.sin()
        cls2 = torch.cat([cls_ang, cls_ang], -1).expand(cls_rows.numel(), -1)
        cls_cos, cls_sin = cls2.cos(), cls2.sin()
        x = self.pre_layernorm(x)
        for blk in self.blocks:
            if self.gradient_checkpointing and self.training:
                x = torch.utils.checkpoint.checkpoint(blk, x, cu, cos, sin, cls_rows, cls_cos, cls_sin, use_reentrant=False)
            else:
                x = blk(x, cu, cos, sin, cls_rows, cls_cos, cls_sin)
        return self.merger(x.index_select(0, keep))
