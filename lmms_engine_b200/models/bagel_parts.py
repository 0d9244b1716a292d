"""Towers around the Bagel decoder: the image autoencoder that gives generation its latents and the packed
variable-resolution SigLIP tower that gives understanding its image tokens.

* ``BagelAutoEncoder`` - the 16-channel, stride-8 latent-diffusion autoencoder (GroupNorm / swish ResNet blocks, one
  single-head attention block in the middle of each half, asymmetric-pad stride-2 convolutions down, nearest x2 +
  convolution up, ``scale * (z - shift)`` on the latents) in the released ``ae.safetensors`` layout
  (src/lmms_engine/models/bagel/autoencoder.py:38-325).
* ``SiglipNavit`` - SigLIP blocks over a PACKED stream of patches from images of any size: patch rows arrive flattened
  (``[n, C*p*p]``, channels last inside a patch, i.e. the released "linear" form of the patch convolution), positions
  are looked up by a flattened ``row * max_side + column`` id (learned table, or 2-D rotary angles on the two halves of
  every head), attention is blind across images through ``cu_seqlens``
  (src/lmms_engine/models/bagel/siglip_navit.py:108-420).
* ``flattened_position_ids`` - the two ways of assigning those ids (extrapolate: plain grid; interpolate: bucketised
  fractional coordinates), src/lmms_engine/models/bagel/data_utils.py:54-70.
"""
from __future__ import annotations

from dataclasses import dataclass, fields
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import attention as attn_ops
from ..ops import gemm as gemm_ops
from ..ops import rope as rope_ops
from .llava_ov import SiglipConfig, _SiglipMLP
from .vision import LayerNorm


# ------------------------------------------------------------------------------------ autoencoder
@dataclass
class AutoEncoderParams:
    resolution: int = 256
    in_channels: int = 3
    downsample: int = 8
    ch: int = 128
    out_ch: int = 3
    ch_mult: Sequence[int] = (1, 2, 4, 4)
    num_res_blocks: int = 2
    z_channels: int = 16
    scale_factor: float = 0.3611
    shift_factor: float = 0.1159

    @classmethod
    def from_dict(cls, d):
        known = {f.name for f in fields(cls)}
        return cls(**{k: v for k, v in (d or {}).items() if k in known})


def _gn(c):
    return nn.GroupNorm(32, c, eps=1e-6, affine=True)


class _AttnBlock(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.norm = _gn(c)
        self.q, self.k, self.v, self.proj_out = (nn.Conv2d(c, c, 1) for _ in range(4))

    def forward(self, x):
        b, c, h, w = x.shape
        y = self.norm(x)
        q, k, v = (m(y).reshape(b, 1, c, h * w).transpose(2, 3) for m in (self.q, self.k, self.v))
        o = F.scaled_dot_product_attention(q, k, v).transpose(2, 3).reshape(b, c, h, w)
        return x + self.proj_out(o)


class _ResnetBlock(nn.Module):
    def __init__(self, c_in, c_out):
        super().__init__()
        self.norm1, self.conv1 = _gn(c_in), nn.Conv2d(c_in, c_out, 3, padding=1)
        self.norm2, self.conv2 = _gn(c_out), nn.Conv2d(c_out, c_out, 3, padding=1)
        if c_in != c_out:
            self.nin_shortcut = nn.Conv2d(c_in, c_out, 1)

    def forward(self, x):
        h = self.conv1(F.silu(self.norm1(x)))
        h = self.conv2(F.silu(self.norm2(h)))
        return (self.nin_shortcut(x) if hasattr(self, "nin_shortcut") else x) + h


class _Down(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.conv = nn.Conv2d(c, c, 3, stride=2, padding=0)

    def forward(self, x):
        return self.conv(F.pad(x, (0, 1, 0, 1)))


class _Up(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.conv = nn.Conv2d(c, c, 3, padding=1)

    def forward(self, x):
        return self.conv(F.interpolate(x, scale_factor=2.0, mode="nearest"))


class _Level(nn.Module):
    pass


class _Mid(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.block_1, self.attn_1, self.block_2 = _ResnetBlock(c, c), _AttnBlock(c), _ResnetBlock(c, c)

    def forward(self, x):
        return self.block_2(self.attn_1(self.block_1(x)))


class _Encoder(nn.Module):
    def __init__(self, p: AutoEncoderParams):
        super().__init__()
        self.conv_in = nn.Conv2d(p.in_channels, p.ch, 3, padding=1)
        mult = (1,) + tuple(p.ch_mult)
        self.down = nn.ModuleList()
        for i in range(len(p.ch_mult)):
            lvl = _Level()
            c_in, c_out = p.ch * mult[i], p.ch * p.ch_mult[i]
            lvl.block = nn.ModuleList([_ResnetBlock(c_in if j == 0 else c_out, c_out) for j in range(p.num_res_blocks)])
            lvl.attn = nn.ModuleList()
            if i != len(p.ch_mult) - 1:
                lvl.downsample = _Down(c_out)
            self.down.append(lvl)
        self.mid = _Mid(c_out)
        self.norm_out, self.conv_out = _gn(c_out), nn.Conv2d(c_out, 2 * p.z_channels, 3, padding=1)

    def forward(self, x):
        h = self.conv_in(x)
        for lvl in self.down:
            for blk in lvl.block:
                h = blk(h)
            if hasattr(lvl, "downsample"):
                h = lvl.downsample(h)
        return self.conv_out(F.silu(self.norm_out(self.mid(h))))


class _Decoder(nn.Module):
    def __init__(self, p: AutoEncoderParams):
        super().__init__()
        n = len(p.ch_mult)
        c = p.ch * p.ch_mult[-1]
        self.conv_in = nn.Conv2d(p.z_channels, c, 3, padding=1)
        self.mid = _Mid(c)
        levels = []
        for i in reversed(range(n)):
            lvl = _Level()
            c_out = p.ch * p.ch_mult[i]
            lvl.block = nn.ModuleList([_ResnetBlock(c if j == 0 else c_out, c_out) for j in range(p.num_res_blocks + 1)])
            lvl.attn = nn.ModuleList()
            c = c_out
            if i != 0:
                lvl.upsample = _Up(c)
            levels.insert(0, lvl)  # stored lowest resolution last, walked in reverse
        self.up = nn.ModuleList(levels)
        self.norm_out, self.conv_out = _gn(c), nn.Conv2d(c, p.out_ch, 3, padding=1)

    def forward(self, z):
        h = self.mid(self.conv_in(z))
        for lvl in reversed(self.up):
            for blk in lvl.block:
                h = blk(h)
            if hasattr(lvl, "upsample"):
                h = lvl.upsample(h)
        return self.conv_out(F.silu(self.norm_out(h)))


class BagelAutoEncoder(nn.Module):
    def __init__(self, params: Optional[AutoEncoderParams] = None, sample: bool = True):
        super().__init__()
        self.params = params or AutoEncoderParams()
        self.encoder, self.decoder = _Encoder(self.params), _Decoder(self.params)
        self.sample = sample

    def encode(self, x: torch.Tensor) -> torch.Tensor:
        mean, logvar = self.encoder(x).chunk(2, 1)
        z = mean + torch.exp(0.5 * logvar) * torch.randn_like(mean) if self.sample else mean
        return self.params.scale_factor * (z - self.params.shift_factor)

    def decode(self, z: torch.Tensor) -> torch.Tensor:
        return self.decoder(z / self.params.scale_factor + self.params.shift_factor)

    def forward(self, x):
        return self.decode(self.encode(x))


# ------------------------------------------------------------------------------------ packed SigLIP
def flattened_position_ids(img_h: int, img_w: int, patch_size: int, max_side: int, interpolate: bool = False) -> torch.Tensor:
    nh, nw = img_h // patch_size, img_w // patch_size
    if not interpolate:
        ch, cw = torch.arange(nh), torch.arange(nw)
    else:
        bounds = torch.arange(1 / max_side, 1.0, 1 / max_side)
        ch = torch.bucketize(torch.arange(0, 1 - 1e-6, 1 / nh), bounds, right=True)
        cw = torch.bucketize(torch.arange(0, 1 - 1e-6, 1 / nw), bounds, right=True)
    return (ch[:, None] * max_side + cw).flatten()


def patchify_image(image: torch.Tensor, patch_size: int) -> torch.Tensor:
    """``[C, H, W] -> [h*w, p*p*C]`` with channels LAST inside a patch (the layout of the linear patch embedding)."""
    C, H, W = image.shape
    p = patch_size
    return image.reshape(C, H // p, p, W // p, p).permute(1, 3, 2, 4, 0).reshape(-1, p * p * C)


class _NavitAttention(nn.Module):
    def __init__(self, d, heads, rope: bool):
        super().__init__()
        self.heads, self.head_dim, self.rope = heads, d // heads, rope
        self.q_proj, self.k_proj, self.v_proj, self.out_proj = (nn.Linear(d, d) for _ in range(4))

    def forward(self, x, cu, cos=None, sin=None):
        P = x.shape[0]
        w = torch.cat([self.q_proj.weight, self.k_proj.weight, self.v_proj.weight], 0)
        b = torch.cat([self.q_proj.bias, self.k_proj.bias, self.v_proj.bias], 0)
        qkv = gemm_ops.linear(x, w, b).view(P, 3, self.heads, self.head_dim)
        q, k, v = qkv[:, 0], qkv[:, 1], qkv[:, 2]
        if self.rope:
            q, k = self._rot(q, cos, sin), self._rot(k, cos, sin)
        o = attn_ops.varlen_attn(q, k, v, cu, cu, causal=False, softmax_scale=self.head_dim ** -0.5)
        return gemm_ops.linear(o.reshape(P, -1), self.out_proj.weight, self.out_proj.bias)

    def _rot(self, x, cos, sin):
        """First half of every head turns with the patch row, second half with the column; each half is a half-split
        rotary of its own (``cos`` / ``sin``: ``[P, 2, D/2]``, row table then column table)."""
        h = x.shape[-1] // 2
        a = rope_ops.rope_apply(x[..., :h], cos[:, 0], sin[:, 0])
        b = rope_ops.rope_apply(x[..., h:], cos[:, 1], sin[:, 1])
        return torch.cat([a, b], -1)


class _NavitLayer(nn.Module):
    def __init__(self, c: SiglipConfig, rope: bool):
        super().__init__()
        self.layer_norm1, self.layer_norm2 = LayerNorm(c.hidden_size, c.layer_norm_eps), LayerNorm(c.hidden_size, c.layer_norm_eps)
        self.self_attn, self.mlp = _NavitAttention(c.hidden_size, c.num_attention_heads, rope), _SiglipMLP(c)

    def forward(self, x, cu, cos=None, sin=None):
        x = x + self.self_attn(self.layer_norm1(x), cu, cos, sin)
        return x + self.mlp(self.layer_norm2(x))


class _NavitEmbeddings(nn.Module):
    def __init__(self, c: SiglipConfig, rope: bool):
        super().__init__()
        self.patch_embedding = nn.Linear(c.num_channels * c.patch_size ** 2, c.hidden_size)
        self.side = c.image_size // c.patch_size
        if not rope:
            self.position_embedding = nn.Embedding(self.side ** 2, c.hidden_size)

    def forward(self, patches, pos_ids):
        x = gemm_ops.linear(patches.to(self.patch_embedding.weight.dtype), self.patch_embedding.weight, self.patch_embedding.bias)
        if hasattr(self, "position_embedding"):
            x = x + self.position_embedding(pos_ids).to(x.dtype)
        return x


class _NavitEncoder(nn.Module):
    def __init__(self, c, rope, layers):
        super().__init__()
        self.layers = nn.ModuleList([_NavitLayer(c, rope) for _ in range(layers)])


class _NavitTransformer(nn.Module):
    def __init__(self, c: SiglipConfig, rope: bool, layers: int):
        super().__init__()
        self.embeddings = _NavitEmbeddings(c, rope)
        self.encoder = _NavitEncoder(c, rope, layers)
        self.post_layernorm = LayerNorm(c.hidden_size, c.layer_norm_eps)


class SiglipNavit(nn.Module):
    """Keys ``vision_model.{embeddings,encoder.layers.N,post_layernorm}`` as released.  ``select_layer`` (negative, like
    the reference's ``vit_select_layer``) drops the last ``-select_layer - 1`` blocks."""

    def __init__(self, c: SiglipConfig, rope: bool = False, select_layer: int = -1):
        super().__init__()
        self.config, self.rope = c, rope
        layers = c.num_hidden_layers + select_layer + 1
        self.vision_model = _NavitTransformer(c, rope, layers)
        self.side = c.image_size // c.patch_size
        self.head_dim = c.hidden_size // c.num_attention_heads

    def load_conv_patch_embedding(self, weight: torch.Tensor, bias: torch.Tensor):
        """A convolutional patch embedding ``[D, C, p, p]`` in its linear form ``[D, p*p*C]`` (channels last)."""
        pe = self.vision_model.embeddings.patch_embedding
        pe.weight.data.copy_(weight.permute(0, 2, 3, 1).reshape(weight.shape[0], -1))
        pe.bias.data.copy_(bias)

    def rotary_tables(self, pos_ids: torch.Tensor):
        d = self.head_dim // 2  # per half
        inv = 1.0 / (10000 ** (torch.arange(0, d, 2, dtype=torch.float32, device=pos_ids.device) / d))
        row, col = (pos_ids // self.side).float(), (pos_ids % self.side).float()
        ang = torch.stack([row[:, None] * inv, col[:, None] * inv], 1)  # [P, 2, d/2]
        ang = torch.cat([ang, ang], -1)  # half-split rotary over d
        return ang.cos(), ang.sin()

    def forward(self, packed_pixel_values, packed_flattened_position_ids, cu_seqlens, max_seqlen: Optional[int] = None):
        vm = self.vision_model
        x = vm.embeddings(packed_pixel_values, packed_flattened_position_ids)
        cos = sin = None
        if self.rope:
            cos, sin = self.rotary_tables(packed_flattened_position_ids)
        for layer in vm.encoder.layers:
            x = layer(x, cu_seqlens, cos, sin)
        return vm.post_layernorm(x)
