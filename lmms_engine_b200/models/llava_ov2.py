"""LLaVA-OneVision-2 family (``model_type: llava_onevision2``): a vision tower that takes every patch
together with its ``(t, h, w)`` position - so images, whole frames and codec-stream videos (only the
patches that changed, see ``datasets/codec_video.py``) are one input format - in front of a Qwen3
decoder on plain 1-D positions.

The reference trains the hub's remote-code implementation and only re-binds its forwards
(src/lmms_engine/models/llava_onevision2/monkey_patch.py:1-266, llava_onevision2_ops.py:58-140): the
contract visible there is ``pixel_values`` + ``image_grid_thw`` + ``patch_positions`` into
``get_image_features``, features written over the image placeholders (videos are aliased into the
image path by the processor), an unpadded Qwen3 decoder and a fused linear + cross-entropy loss.
This module implements that contract natively on the engine's packed kernels; the tower's internals
(pre-LayerNorm, LayerNorm blocks with fused qkv, 3-D rotary angles read from ``patch_positions``,
LayerNorm + two-layer GELU merger over ``merge x merge`` blocks) are this engine's own, since the remote
code is not part of the reference tree.  There is therefore no hub-name mapping for the tower.
"""
from __future__ import annotations

import math
from typing import Optional

import numpy as np
import torch
import torch.nn as nn

from ..ops import attention as attn_ops
from ..ops import gemm as gemm_ops
from ..ops import rope as rope_ops
from .rice import RiceMLP, RiceMerger, RicePatchEmbed
from .vision import LayerNorm, VisionConfig, _grid_list
from .vl import VLModel


def rotary_sections(half: int):
    """Split of the ``head_dim / 2`` rotary frequencies between time, height and width (2 : 3 : 3)."""
    hw = (half * 3) // 8
    return half - 2 * hw, hw, hw


class OV2Attention(nn.Module):
    def __init__(self, dim: int, heads: int):
        super().__init__()
        self.heads, self.head_dim = heads, dim // heads
        self.qkv = nn.Linear(dim, dim * 3, bias=True)
        self.proj = nn.Linear(dim, dim)

    def forward(self, x, cu, cos, sin):
        P = x.shape[0]
        qkv = gemm_ops.linear(x, self.qkv.weight, self.qkv.bias).view(P, 3, self.heads, self.head_dim)
        q = rope_ops.rope_apply(qkv[:, 0], cos, sin)
        k = rope_ops.rope_apply(qkv[:, 1], cos, sin)
        o = attn_ops.varlen_attn(q, k, qkv[:, 2], cu, cu, causal=False, softmax_scale=1.0 / math.sqrt(self.head_dim))
        return gemm_ops.linear(o.reshape(P, -1), self.proj.weight, self.proj.bias)


class OV2Block(nn.Module):
    def __init__(self, cfg: VisionConfig):
        super().__init__()
        self.norm1 = LayerNorm(cfg.hidden_size, 1e-5)
        self.norm2 = LayerNorm(cfg.hidden_size, 1e-5)
        self.attn = OV2Attention(cfg.hidden_size, cfg.num_heads)
        self.mlp = RiceMLP(cfg.hidden_size, cfg.intermediate_size, cfg.hidden_act)

    def forward(self, x, cu, cos, sin):
        x = x + self.attn(self.norm1(x), cu, cos, sin)
        return x + self.mlp(self.norm2(x))


class OneVisionTower(nn.Module):
    """``forward(patches [N, C*p*p], grid_thw [n, 3], patch_positions [N, 3])`` -> ``[N / merge^2, out_hidden]``.
    The patches of entry ``i`` are ``t*h*w`` consecutive rows in block layout (the ``merge^2`` patches of a merged
    token adjacent); attention is full inside an entry and blind across entries."""

    def __init__(self, cfg: VisionConfig):
        super().__init__()
        self.cfg = cfg
        eps = float(cfg.extra.get("layer_norm_eps", 1e-5))
        self.patch_embed = RicePatchEmbed(cfg)
        self.layernorm_pre = LayerNorm(cfg.hidden_size, eps)
        self.blocks = nn.ModuleList([OV2Block(cfg) for _ in range(cfg.depth)])
        self.merger = RiceMerger(cfg.out_hidden_size, cfg.hidden_size, cfg.spatial_merge_size, eps)
        self.gradient_checkpointing = False
        self.rope_theta = float(cfg.extra.get("rope_theta", 10000.0))
        for m in self.modules():
            if isinstance(m, (nn.Linear, nn.Conv2d)):
                nn.init.normal_(m.weight, 0.0, cfg.initializer_range)
                if m.bias is not None:
                    nn.init.zeros_(m.bias)

    def angles(self, positions: torch.Tensor) -> torch.Tensor:
        """Rotary angles ``[N, head_dim / 2]``: the first section turns with t, the second with h, the third with w."""
        half = self.cfg.hidden_size // self.cfg.num_heads // 2
        parts = []
        for axis, n in enumerate(rotary_sections(half)):
            invf = 1.0 / (self.rope_theta ** (torch.arange(n, dtype=torch.float32, device=positions.device) / max(n, 1)))
            parts.append(positions[:, axis:axis + 1].float() * invf[None])
        return torch.cat(parts, -1)

    def forward(self, patches: torch.Tensor, grid_thw, patch_positions: Optional[torch.Tensor] = None) -> torch.Tensor:
        grid = _grid_list(grid_thw)
        dev = patches.device
        counts = [t * h * w for t, h, w in grid]
        if sum(counts) != patches.shape[0]:
            raise ValueError(f"grids describe {sum(counts)} patches, got {patches.shape[0]}")
        if patch_positions is None:
            patch_positions = getattr(self, "pending_positions", None)  # set by the model around its forward
        if patch_positions is None:
            patch_positions = torch.from_numpy(build_patch_positions(grid, self.cfg.spatial_merge_size)).to(dev)
        if patch_positions.shape[0] != patches.shape[0]:
            raise ValueError(f"{patch_positions.shape[0]} patch positions for {patches.shape[0]} patches")
        cu = torch.from_numpy(np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)).to(dev, non_blocking=True)
        ang = self.angles(patch_positions.to(dev))
        full = torch.cat([ang, ang], -1)
        cos, sin = full.cos(), full.sin()
        x = self.layernorm_pre(self.patch_embed(patches))
        for blk in self.blocks:
            if self.gradient_checkpointing and self.training:
                x = torch.utils.checkpoint.checkpoint(blk, x, cu, cos, sin, use_reentrant=False)
            else:
                x = blk(x, cu, cos, sin)
        return self.merger(x)


def build_patch_positions(grid, merge: int) -> np.ndarray:
    """``(t, h, w)`` of every patch of full frames in block layout (what an image or a plainly sampled video has)."""
    out = []
    for t, h, w in grid:
        tt, hh, ww = np.meshgrid(np.arange(t), np.arange(h), np.arange(w), indexing="ij")
        pos = np.stack([tt, hh, ww], -1)  # t, h, w, 3
        pos = pos.reshape(t, h // merge, merge, w // merge, merge, 3).transpose(0, 1, 3, 2, 4, 5).reshape(-1, 3)
        out.append(pos)
    return np.concatenate(out, 0) if out else np.zeros((0, 3), np.int64)


class LlavaOnevision2(VLModel):
    """``VLModel`` whose tower receives ``patch_positions`` next to the patches; videos arrive through the image
    inputs (the processor aliases them), so ``pixel_values_videos`` is accepted only as a synonym."""

    def forward(self, patch_positions=None, pixel_values=None, image_grid_thw=None, pixel_values_videos=None, video_grid_thw=None, **kw):
        if pixel_values is None and pixel_values_videos is not None:
            pixel_values, image_grid_thw = pixel_values_videos, video_grid_thw
        self.visual.pending_positions = patch_positions
        try:
            return super().forward(pixel_values=pixel_values, image_grid_thw=image_grid_thw, **kw)
        finally:
            self.visual.pending_positions = None
