"""Frozen condition encoders of the Wan video family and its small add-on controllers.

* ``WanTextEncoder`` - the umT5 encoder (pre-RMSNorm blocks, unscaled attention with a learned relative-position
  bias PER LAYER, gated tanh-GELU feed-forward).  Parameter names are those of the released ``umt5-xxl`` encoder
  checkpoint (``token_embedding``, ``blocks.N.{norm1,attn.{q,k,v,o},pos_embedding.embedding,norm2,ffn.{gate.0,fc1,fc2}}``,
  ``norm``); reference: src/lmms_engine/models/wanvideo/wan_video_text_encoder.py:20-245.
* ``WanImageEncoder`` - the vision tower of the XLM-R CLIP ViT-H/14 (class token, learned positions, pre-norm, GELU
  blocks); ``encode_image`` returns the token states after all blocks but the last, which is what the DiT's image
  branch consumes; reference: wan_video_image_encoder.py:387-494, 872-894.
* ``WanMotionController`` - motion-bucket id -> additive timestep modulation (wan_video_motion_controller.py:7-28).

Projections run on the engine's GEMM; the relative-position bias keeps T5 attention on the framework's attention
with an additive mask (a frozen encoder, evaluated once per sample).
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import attention as attn_ops
from ..ops import gemm as gemm_ops
from .vision import LayerNorm


def sinusoid_1d(dim: int, position: torch.Tensor) -> torch.Tensor:
    """``[n] -> [n, dim]``: cosines then sines of ``position / 10000^(i / (dim/2))`` (fp64 inside)."""
    inv = torch.pow(10000.0, -torch.arange(dim // 2, dtype=torch.float64, device=position.device) / (dim // 2))
    ang = torch.outer(position.to(torch.float64), inv)
    return torch.cat([ang.cos(), ang.sin()], 1).to(position.dtype if position.is_floating_point() else torch.float32)


# ------------------------------------------------------------------------------------ umT5 encoder
class T5Norm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6):
        super().__init__()
        self.weight, self.eps = nn.Parameter(torch.ones(dim)), eps

    def forward(self, x):
        y = x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + self.eps)
        return self.weight * y.to(self.weight.dtype)


class T5RelativeBias(nn.Module):
    """Bidirectional bucketed relative positions: half of the buckets for keys after the query, half for keys before;
    within a half, exact up to ``n/2`` then logarithmic up to ``max_dist``."""

    def __init__(self, num_buckets: int, num_heads: int, max_dist: int = 128):
        super().__init__()
        self.num_buckets, self.max_dist = num_buckets, max_dist
        self.embedding = nn.Embedding(num_buckets, num_heads)

    def buckets(self, lq: int, lk: int, device) -> torch.Tensor:
        rel = torch.arange(lk, device=device)[None] - torch.arange(lq, device=device)[:, None]
        n = self.num_buckets // 2
        out = (rel > 0).long() * n
        rel = rel.abs()
        exact = n // 2
        large = exact + (torch.log(rel.float().clamp(min=1) / exact) / math.log(self.max_dist / exact) * (n - exact)).long()
        return out + torch.where(rel < exact, rel, large.clamp(max=n - 1))

    def forward(self, lq: int, lk: int) -> torch.Tensor:
        return self.embedding(self.buckets(lq, lk, self.embedding.weight.device)).permute(2, 0, 1)[None]  # [1, heads, lq, lk]


class _T5Attention(nn.Module):
    def __init__(self, dim, dim_attn, heads):
        super().__init__()
        self.heads, self.head_dim = heads, dim_attn // heads
        self.q, self.k, self.v = (nn.Linear(dim, dim_attn, bias=False) for _ in range(3))
        self.o = nn.Linear(dim_attn, dim, bias=False)

    def forward(self, x, bias):  # x [B, L, C], bias [B or 1, heads, L, L] additive
        B, L, _ = x.shape
        w = torch.cat([self.q.weight, self.k.weight, self.v.weight], 0)
        qkv = gemm_ops.linear(x.reshape(B * L, -1), w, None).view(B, L, 3, self.heads, self.head_dim).permute(2, 0, 3, 1, 4)
        o = F.scaled_dot_product_attention(qkv[0], qkv[1], qkv[2], attn_mask=bias.to(x.dtype), scale=1.0)  # T5: no 1/sqrt(d)
        return gemm_ops.linear(o.transpose(1, 2).reshape(B * L, -1), self.o.weight, None).view(B, L, -1)


class _T5FeedForward(nn.Module):
    def __init__(self, dim, dim_ffn):
        super().__init__()
        self.gate = nn.Sequential(nn.Linear(dim, dim_ffn, bias=False), nn.GELU(approximate="tanh"))
        self.fc1, self.fc2 = nn.Linear(dim, dim_ffn, bias=False), nn.Linear(dim_ffn, dim, bias=False)

    def forward(self, x):
        shape = x.shape
        x = x.reshape(-1, shape[-1])
        h = gemm_ops.linear(x, self.fc1.weight, None) * F.gelu(gemm_ops.linear(x, self.gate[0].weight, None), approximate="tanh")
        return gemm_ops.linear(h, self.fc2.weight, None).view(shape)


class _T5Block(nn.Module):
    def __init__(self, dim, dim_attn, dim_ffn, heads, buckets, shared_pos):
        super().__init__()
        self.norm1, self.norm2 = T5Norm(dim), T5Norm(dim)
        self.attn, self.ffn = _T5Attention(dim, dim_attn, heads), _T5FeedForward(dim, dim_ffn)
        self.pos_embedding = None if shared_pos else T5RelativeBias(buckets, heads)

    def forward(self, x, mask_bias, shared_bias):
        pos = shared_bias if self.pos_embedding is None else self.pos_embedding(x.shape[1], x.shape[1])
        x = x + self.attn(self.norm1(x), pos + mask_bias)
        return x + self.ffn(self.norm2(x))


class WanTextEncoder(nn.Module):
    def __init__(self, vocab: int = 256384, dim: int = 4096, dim_attn: int = 4096, dim_ffn: int = 10240, num_heads: int = 64,
                 num_layers: int = 24, num_buckets: int = 32, shared_pos: bool = False):
        super().__init__()
        self.dim = dim
        self.token_embedding = nn.Embedding(vocab, dim)
        self.pos_embedding = T5RelativeBias(num_buckets, num_heads) if shared_pos else None
        self.blocks = nn.ModuleList([_T5Block(dim, dim_attn, dim_ffn, num_heads, num_buckets, shared_pos) for _ in range(num_layers)])
        self.norm = T5Norm(dim)
        for m in self.modules():
            if isinstance(m, nn.Linear):
                nn.init.normal_(m.weight, std=m.in_features ** -0.5)
            elif isinstance(m, T5RelativeBias):
                nn.init.normal_(m.embedding.weight, std=(2 * num_buckets * num_heads) ** -0.5)

    def forward(self, ids: torch.Tensor, mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``ids [B, L]``, ``mask [B, L]`` (1 = token) -> ``[B, L, dim]``."""
        x = self.token_embedding(ids)
        B, L, _ = x.shape
        mask_bias = x.new_zeros((B, 1, 1, L), dtype=torch.float32)
        if mask is not None:
            mask_bias = mask_bias.masked_fill(mask.view(B, 1, 1, L) == 0, torch.finfo(torch.float32).min / 2)
        shared = self.pos_embedding(L, L) if self.pos_embedding is not None else None
        for blk in self.blocks:
            x = blk(x, mask_bias, shared)
        return self.norm(x)

    def encode_prompt(self, ids: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
        """Prompt embedding with the rows of padding tokens zeroed."""
        return self.forward(ids, mask) * (mask > 0).unsqueeze(-1).to(self.norm.weight.dtype)


# ------------------------------------------------------------------------------------ CLIP vision tower
CLIP_MEAN = (0.48145466, 0.4578275, 0.40821073)
CLIP_STD = (0.26862954, 0.26130258, 0.27577711)


class _ClipAttention(nn.Module):
    def __init__(self, dim, heads):
        super().__init__()
        self.heads, self.head_dim = heads, dim // heads
        self.to_qkv, self.proj = nn.Linear(dim, 3 * dim), nn.Linear(dim, dim)

    def forward(self, x, cu):
        P = x.shape[0]
        qkv = gemm_ops.linear(x, self.to_qkv.weight, self.to_qkv.bias).view(P, 3, self.heads, self.head_dim)
        o = attn_ops.varlen_attn(qkv[:, 0], qkv[:, 1], qkv[:, 2], cu, cu, causal=False, softmax_scale=self.head_dim ** -0.5)
        return gemm_ops.linear(o.reshape(P, -1), self.proj.weight, self.proj.bias)


class _ClipBlock(nn.Module):
    def __init__(self, dim, ratio, heads, activation, eps):
        super().__init__()
        self.norm1, self.norm2 = LayerNorm(dim, eps), LayerNorm(dim, eps)
        self.attn = _ClipAttention(dim, heads)
        self.activation = activation
        self.mlp = nn.Sequential(nn.Linear(dim, int(dim * ratio)), nn.Identity(), nn.Linear(int(dim * ratio), dim))

    def forward(self, x, cu):
        x = x + self.attn(self.norm1(x), cu)
        h = gemm_ops.linear(self.norm2(x), self.mlp[0].weight, self.mlp[0].bias)
        h = h * torch.sigmoid(1.702 * h) if self.activation == "quick_gelu" else F.gelu(h)
        return x + gemm_ops.linear(h, self.mlp[2].weight, self.mlp[2].bias)


class ClipVisionTower(nn.Module):
    def __init__(self, image_size=224, patch_size=14, dim=1280, mlp_ratio=4, out_dim=1024, num_heads=16, num_layers=32,
                 activation="gelu", norm_eps=1e-5):
        super().__init__()
        self.image_size, self.patch_size, self.dim = image_size, patch_size, dim
        n = (image_size // patch_size) ** 2
        gain = 1.0 / math.sqrt(dim)
        self.patch_embedding = nn.Conv2d(3, dim, patch_size, patch_size, bias=False)
        self.cls_embedding = nn.Parameter(gain * torch.randn(1, 1, dim))
        self.pos_embedding = nn.Parameter(gain * torch.randn(1, n + 1, dim))
        self.pre_norm = LayerNorm(dim, norm_eps)
        self.transformer = nn.ModuleList([_ClipBlock(dim, mlp_ratio, num_heads, activation, norm_eps) for _ in range(num_layers)])
        self.post_norm = LayerNorm(dim, norm_eps)
        self.head = nn.Parameter(gain * torch.randn(dim, out_dim))

    def forward(self, x: torch.Tensor, skip_last_block: bool = False) -> torch.Tensor:
        """``[B, 3, S, S]`` -> token states ``[B, 1 + n, dim]`` (no post-norm, no projection head)."""
        B, p = x.shape[0], self.patch_size
        side = x.shape[-1] // p
        w = self.patch_embedding.weight
        rows = x.reshape(B, 3, side, p, side, p).permute(0, 2, 4, 1, 3, 5).reshape(B * side * side, 3 * p * p)
        tok = gemm_ops.linear(rows.to(w.dtype), w.view(w.shape[0], -1), None).view(B, side * side, -1)
        tok = torch.cat([self.cls_embedding.expand(B, -1, -1).to(tok.dtype), tok], 1) + self.pos_embedding.to(tok.dtype)
        n = tok.shape[1]
        h = self.pre_norm(tok.reshape(B * n, -1))
        cu = (torch.arange(B + 1, device=h.device) * n).to(torch.int32)
        blocks = self.transformer[:-1] if skip_last_block else self.transformer
        for blk in blocks:
            h = blk(h, cu)
        return h.view(B, n, -1)


class _ClipHolder(nn.Module):
    def __init__(self, **kw):
        super().__init__()
        self.visual = ClipVisionTower(**kw)


class WanImageEncoder(nn.Module):
    """Keys ``model.visual.*`` as in the released CLIP checkpoint; its text half is not part of the video model."""

    def __init__(self, **kw):
        super().__init__()
        self.model = _ClipHolder(**kw)
        self.register_buffer("mean", torch.tensor(CLIP_MEAN).view(1, 3, 1, 1), persistent=False)
        self.register_buffer("std", torch.tensor(CLIP_STD).view(1, 3, 1, 1), persistent=False)

    @torch.no_grad()
    def encode_image(self, images: Sequence[torch.Tensor]) -> torch.Tensor:
        """Images in ``[-1, 1]`` (each ``[b, 3, H, W]``) -> ``[sum b, 257, 1280]`` states before the last block."""
        S = self.model.visual.image_size
        x = torch.cat([F.interpolate(u.float(), size=(S, S), mode="bicubic", align_corners=False) for u in images])
        x = ((x * 0.5 + 0.5) - self.mean) / self.std
        return self.model.visual(x.to(self.model.visual.patch_embedding.weight.dtype), skip_last_block=True)

    def convert_state_dict(self, sd):
        """Drop the text half (``model.textual.*``, ``model.log_scale``) of a full CLIP checkpoint."""
        return {k: v for k, v in sd.items() if k.startswith("model.visual.")}


# ------------------------------------------------------------------------------------ motion controller
class WanMotionController(nn.Module):
    def __init__(self, freq_dim: int = 256, dim: int = 1536):
        super().__init__()
        self.freq_dim = freq_dim
        self.linear = nn.Sequential(nn.Linear(freq_dim, dim), nn.SiLU(), nn.Linear(dim, dim), nn.SiLU(), nn.Linear(dim, dim * 6))
        nn.init.zeros_(self.linear[-1].weight)
        nn.init.zeros_(self.linear[-1].bias)  # starts as "no change" to the timestep modulation

    def forward(self, motion_bucket_id: torch.Tensor) -> torch.Tensor:
        return self.linear(sinusoid_1d(self.freq_dim, motion_bucket_id.float() * 10).to(self.linear[0].weight.dtype))
