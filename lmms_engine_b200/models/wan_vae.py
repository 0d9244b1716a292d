"""Causal 3-D video autoencoders of the Wan family: the 16-channel one (stride 4 x 8 x 8) and the 48-channel one
(input folded 2 x 2 into channels, stride 4 x 16 x 16, averaging / duplicating shortcuts around every stage).

The released implementations walk a video in chunks (first frame alone, then four frames at a time; one latent
frame at a time when decoding) and carry the last frames of every convolution's input from chunk to chunk
(src/lmms_engine/models/wanvideo/wan_video_vae.py:31-56, 82-167, 247-286, 496-606, 718-831, 948-1058, 1340-1438).
Here the whole sequence is processed at once; the chunk protocol fixes three facts that the whole-sequence form
has to reproduce, and does:

* every 3-tap temporal convolution is causal with zero history (pad two frames in front);
* a temporal down-sampling stage passes the FIRST frame through untouched and runs its stride-2 convolution,
  unpadded, over the full sequence (frame 0 included) for the rest: ``T -> 1 + (T - 1) / 2``;
* a temporal up-sampling stage passes the first frame through untouched and doubles every later frame with a causal
  convolution whose history starts at frame 1 (frame 0 is not part of it): ``T -> 1 + 2 (T - 1)``.

Module and parameter names are the released checkpoints' (``model.encoder.downsamples.N.residual.2.weight`` ...), kept by
building every ``nn.Sequential`` with the same slots.  Convolutions are library calls (cuDNN): the autoencoder is a
frozen pre-/post-processor of the diffusion transformer, not part of its training step's hot loop.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

WAN21_MEAN = [-0.7571, -0.7089, -0.9113, 0.1075, -0.1745, 0.9653, -0.1517, 1.5508, 0.4134, -0.0715, 0.5517, -0.3632, -0.1922, -0.9497,
              0.2503, -0.2921]
WAN21_STD = [2.8184, 1.4541, 2.3275, 2.6558, 1.2196, 1.7708, 2.6052, 2.0743, 3.2687, 2.1526, 2.8652, 1.5579, 1.6382, 1.1253, 2.8251,
             1.9160]


class CausalConv3d(nn.Conv3d):
    """3-D convolution that pads time only in front (twice the symmetric amount), space symmetrically."""

    def __init__(self, *a, **k):
        super().__init__(*a, **k)
        pt, ph, pw = self.padding
        self._pad = (pw, pw, ph, ph, 2 * pt, 0)
        self.padding = (0, 0, 0)

    def forward(self, x):
        return super().forward(F.pad(x, self._pad))


class ChannelRmsNorm(nn.Module):
    """Unit-normalise over channels (dim 1), times ``sqrt(C)`` and a per-channel gain."""

    def __init__(self, dim: int, images: bool = True):
        super().__init__()
        self.scale = dim ** 0.5
        self.gamma = nn.Parameter(torch.ones((dim, 1, 1) if images else (dim, 1, 1, 1)))

    def forward(self, x):
        return F.normalize(x, dim=1) * self.scale * self.gamma


class _Up2x(nn.Module):
    def forward(self, x):
        return F.interpolate(x.float(), scale_factor=(2.0, 2.0), mode="nearest-exact").type_as(x)


def _per_frame(fn, x):
    b, c, t, h, w = x.shape
    y = fn(x.permute(0, 2, 1, 3, 4).reshape(b * t, c, h, w))
    return y.view(b, t, *y.shape[1:]).permute(0, 2, 1, 3, 4)


class Resample(nn.Module):
    """Spatial x2 up / down per frame, with the temporal halves described in the module docstring for the 3-D modes.
    ``halve``: the up-sampling convolution also halves the channels (16-channel autoencoder)."""

    def __init__(self, dim: int, mode: str, halve: bool = True):
        super().__init__()
        self.mode = mode
        if mode in ("upsample2d", "upsample3d"):
            self.resample = nn.Sequential(_Up2x(), nn.Conv2d(dim, dim // 2 if halve else dim, 3, padding=1))
            if mode == "upsample3d":
                self.time_conv = CausalConv3d(dim, dim * 2, (3, 1, 1), padding=(1, 0, 0))
        elif mode in ("downsample2d", "downsample3d"):
            self.resample = nn.Sequential(nn.ZeroPad2d((0, 1, 0, 1)), nn.Conv2d(dim, dim, 3, stride=(2, 2)))
            if mode == "downsample3d":
                self.time_conv = CausalConv3d(dim, dim, (3, 1, 1), stride=(2, 1, 1), padding=(0, 0, 0))
        else:
            raise ValueError(mode)

    def forward(self, x):
        if self.mode == "upsample3d" and x.shape[2] > 1:
            b, c, t, h, w = x.shape
            r = self.time_conv(x[:, :, 1:]).view(b, 2, c, t - 1, h, w)
            r = torch.stack((r[:, 0], r[:, 1]), 3).reshape(b, c, 2 * (t - 1), h, w)  # frame 2i from the first half, 2i+1 from the second
            x = torch.cat([x[:, :, :1], r], 2)
        x = _per_frame(self.resample, x)
        if self.mode == "downsample3d" and x.shape[2] > 1:
            x = torch.cat([x[:, :, :1], self.time_conv(x)], 2)
        return x


class ResidualBlock(nn.Module):
    def __init__(self, in_dim: int, out_dim: int, dropout: float = 0.0):
        super().__init__()
        self.residual = nn.Sequential(ChannelRmsNorm(in_dim, images=False), nn.SiLU(), CausalConv3d(in_dim, out_dim, 3, padding=1),
                                      ChannelRmsNorm(out_dim, images=False), nn.SiLU(), nn.Dropout(dropout),
                                      CausalConv3d(out_dim, out_dim, 3, padding=1))
        self.shortcut = CausalConv3d(in_dim, out_dim, 1) if in_dim != out_dim else nn.Identity()

    def forward(self, x):
        return self.residual(x) + self.shortcut(x)


class AttentionBlock(nn.Module):
    """Single-head attention over the pixels of each frame (frames do not see each other)."""

    def __init__(self, dim: int):
        super().__init__()
        self.norm = ChannelRmsNorm(dim)
        self.to_qkv, self.proj = nn.Conv2d(dim, dim * 3, 1), nn.Conv2d(dim, dim, 1)
        nn.init.zeros_(self.proj.weight)

    def _frame(self, x):
        n, c, h, w = x.shape
        q, k, v = self.to_qkv(self.norm(x)).reshape(n, 1, 3 * c, h * w).transpose(2, 3).chunk(3, -1)
        o = F.scaled_dot_product_attention(q, k, v)
        return self.proj(o.squeeze(1).transpose(1, 2).reshape(n, c, h, w))

    def forward(self, x):
        return x + _per_frame(self._frame, x)


def _run(seq, x):
    for m in seq:
        x = m(x)
    return x


class Encoder3d(nn.Module):
    def __init__(self, dim=96, z_dim=32, dim_mult=(1, 2, 4, 4), num_res_blocks=2, attn_scales=(), temporal_downsample=(False, True, True),
                 dropout=0.0, in_channels=3):
        super().__init__()
        dims = [dim * u for u in (1,) + tuple(dim_mult)]
        scale = 1.0
        self.conv1 = CausalConv3d(in_channels, dims[0], 3, padding=1)
        blocks: List[nn.Module] = []
        for i, (a, b) in enumerate(zip(dims[:-1], dims[1:])):
            for _ in range(num_res_blocks):
                blocks.append(ResidualBlock(a, b, dropout))
                if scale in attn_scales:
                    blocks.append(AttentionBlock(b))
                a = b
            if i != len(dim_mult) - 1:
                blocks.append(Resample(b, "downsample3d" if temporal_downsample[i] else "downsample2d"))
                scale /= 2.0
        self.downsamples = nn.Sequential(*blocks)
        self.middle = nn.Sequential(ResidualBlock(b, b, dropout), AttentionBlock(b), ResidualBlock(b, b, dropout))
        self.head = nn.Sequential(ChannelRmsNorm(b, images=False), nn.SiLU(), CausalConv3d(b, z_dim, 3, padding=1))

    def forward(self, x):
        return self.head(self.middle(self.downsamples(self.conv1(x))))


class Decoder3d(nn.Module):
    def __init__(self, dim=96, z_dim=16, dim_mult=(1, 2, 4, 4), num_res_blocks=2, attn_scales=(), temporal_upsample=(True, True, False),
                 dropout=0.0, out_channels=3):
        super().__init__()
        dims = [dim * u for u in (dim_mult[-1],) + tuple(dim_mult[::-1])]
        scale = 1.0 / 2 ** (len(dim_mult) - 2)
        self.conv1 = CausalConv3d(z_dim, dims[0], 3, padding=1)
        self.middle = nn.Sequential(ResidualBlock(dims[0], dims[0], dropout), AttentionBlock(dims[0]), ResidualBlock(dims[0], dims[0], dropout))
        blocks: List[nn.Module] = []
        for i, (a, b) in enumerate(zip(dims[:-1], dims[1:])):
            if i in (1, 2, 3):
                a = a // 2  # the previous stage's up-sampling convolution halved the channels
            for _ in range(num_res_blocks + 1):
                blocks.append(ResidualBlock(a, b, dropout))
                if scale in attn_scales:
                    blocks.append(AttentionBlock(b))
                a = b
            if i != len(dim_mult) - 1:
                blocks.append(Resample(b, "upsample3d" if temporal_upsample[i] else "upsample2d"))
                scale *= 2.0
        self.upsamples = nn.Sequential(*blocks)
        self.head = nn.Sequential(ChannelRmsNorm(b, images=False), nn.SiLU(), CausalConv3d(b, out_channels, 3, padding=1))

    def forward(self, x):
        return self.head(self.upsamples(self.middle(self.conv1(x))))


# ---- 48-channel variant -----------------------------------------------------------------------------------------
class AvgDown3D(nn.Module):
    """Parameter-free shortcut of a down stage: fold ``factor_t x factor_s x factor_s`` neighbours into channels and
    average groups of channels down to ``out_channels``; time is padded in FRONT to a multiple of ``factor_t``."""

    def __init__(self, in_channels, out_channels, factor_t, factor_s=1):
        super().__init__()
        self.out_channels, self.ft, self.fs = out_channels, factor_t, factor_s
        self.factor = factor_t * factor_s * factor_s
        assert in_channels * self.factor % out_channels == 0
        self.group = in_channels * self.factor // out_channels

    def forward(self, x):
        x = F.pad(x, (0, 0, 0, 0, (self.ft - x.shape[2] % self.ft) % self.ft, 0))
        B, C, T, H, W = x.shape
        ft, fs = self.ft, self.fs
        x = x.view(B, C, T // ft, ft, H // fs, fs, W // fs, fs).permute(0, 1, 3, 5, 7, 2, 4, 6)
        return x.reshape(B, self.out_channels, self.group, T // ft, H // fs, W // fs).mean(2)


class DupUp3D(nn.Module):
    """Parameter-free shortcut of an up stage: repeat channels and unfold them into ``factor_t x factor_s x factor_s``
    neighbours; the frames that the duplicated FIRST frame would add in front are dropped."""

    def __init__(self, in_channels, out_channels, factor_t, factor_s=1):
        super().__init__()
        self.out_channels, self.ft, self.fs = out_channels, factor_t, factor_s
        assert out_channels * factor_t * factor_s * factor_s % in_channels == 0
        self.repeats = out_channels * factor_t * factor_s * factor_s // in_channels

    def forward(self, x):
        B, _, T, H, W = x.shape
        ft, fs = self.ft, self.fs
        x = x.repeat_interleave(self.repeats, 1).view(B, self.out_channels, ft, fs, fs, T, H, W).permute(0, 1, 5, 2, 6, 3, 7, 4)
        return x.reshape(B, self.out_channels, T * ft, H * fs, W * fs)[:, :, ft - 1:]


class DownResidualBlock(nn.Module):
    def __init__(self, in_dim, out_dim, dropout, mult, temporal_downsample=False, down_flag=False):
        super().__init__()
        self.avg_shortcut = AvgDown3D(in_dim, out_dim, 2 if temporal_downsample else 1, 2 if down_flag else 1)
        blocks: List[nn.Module] = []
        for _ in range(mult):
            blocks.append(ResidualBlock(in_dim, out_dim, dropout))
            in_dim = out_dim
        if down_flag:
            blocks.append(Resample(out_dim, "downsample3d" if temporal_downsample else "downsample2d", halve=False))
        self.downsamples = nn.Sequential(*blocks)

    def forward(self, x):
        return self.downsamples(x) + self.avg_shortcut(x)


class UpResidualBlock(nn.Module):
    def __init__(self, in_dim, out_dim, dropout, mult, temporal_upsample=False, up_flag=False):
        super().__init__()
        self.avg_shortcut = DupUp3D(in_dim, out_dim, 2 if temporal_upsample else 1, 2) if up_flag else None
        blocks: List[nn.Module] = []
        for _ in range(mult):
            blocks.append(ResidualBlock(in_dim, out_dim, dropout))
            in_dim = out_dim
        if up_flag:
            blocks.append(Resample(out_dim, "upsample3d" if temporal_upsample else "upsample2d", halve=False))
        self.upsamples = nn.Sequential(*blocks)

    def forward(self, x):
        y = self.upsamples(x)
        return y if self.avg_shortcut is None else y + self.avg_shortcut(x)


class Encoder3d38(nn.Module):
    def __init__(self, dim=160, z_dim=96, dim_mult=(1, 2, 4, 4), num_res_blocks=2, temporal_downsample=(False, True, True), dropout=0.0):
        super().__init__()
        dims = [dim * u for u in (1,) + tuple(dim_mult)]
        self.conv1 = CausalConv3d(12, dims[0], 3, padding=1)
        stages = []
        for i, (a, b) in enumerate(zip(dims[:-1], dims[1:])):
            t_down = temporal_downsample[i] if i < len(temporal_downsample) else False
            stages.append(DownResidualBlock(a, b, dropout, num_res_blocks, t_down, i != len(dim_mult) - 1))
        self.downsamples = nn.Sequential(*stages)
        self.middle = nn.Sequential(ResidualBlock(b, b, dropout), AttentionBlock(b), ResidualBlock(b, b, dropout))
        self.head = nn.Sequential(ChannelRmsNorm(b, images=False), nn.SiLU(), CausalConv3d(b, z_dim, 3, padding=1))

    def forward(self, x):
        return self.head(self.middle(self.downsamples(self.conv1(x))))


class Decoder3d38(nn.Module):
    def __init__(self, dim=256, z_dim=48, dim_mult=(1, 2, 4, 4), num_res_blocks=2, temporal_upsample=(True, True, False), dropout=0.0):
        super().__init__()
        dims = [dim * u for u in (dim_mult[-1],) + tuple(dim_mult[::-1])]
        self.conv1 = CausalConv3d(z_dim, dims[0], 3, padding=1)
        self.middle = nn.Sequential(ResidualBlock(dims[0], dims[0], dropout), AttentionBlock(dims[0]), ResidualBlock(dims[0], dims[0], dropout))
        stages = []
        for i, (a, b) in enumerate(zip(dims[:-1], dims[1:])):
            t_up = temporal_upsample[i] if i < len(temporal_upsample) else False
            stages.append(UpResidualBlock(a, b, dropout, num_res_blocks + 1, t_up, i != len(dim_mult) - 1))
        self.upsamples = nn.Sequential(*stages)
        self.head = nn.Sequential(ChannelRmsNorm(b, images=False), nn.SiLU(), CausalConv3d(b, 12, 3, padding=1))

    def forward(self, x):
        return self.head(self.upsamples(self.middle(self.conv1(x))))


def fold2x2(x):
    """``[b, c, f, 2h, 2w] -> [b, 4c, f, h, w]`` with channel order (c, column offset, row offset)."""
    b, c, f, H, W = x.shape
    return x.view(b, c, f, H // 2, 2, W // 2, 2).permute(0, 1, 6, 4, 2, 3, 5).reshape(b, c * 4, f, H // 2, W // 2)


def unfold2x2(x):
    b, C, f, h, w = x.shape
    return x.view(b, C // 4, 2, 2, f, h, w).permute(0, 1, 4, 5, 3, 6, 2).reshape(b, C // 4, f, h * 2, w * 2)


# ---- wrappers ---------------------------------------------------------------------------------------------------
class VideoVAE(nn.Module):
    """``encode`` returns the normalised posterior mean, ``decode`` inverts the normalisation first."""

    def __init__(self, variant: str = "wan2.1", dim: Optional[int] = None, z_dim: Optional[int] = None, dec_dim: Optional[int] = None,
                 dim_mult=(1, 2, 4, 4), num_res_blocks: int = 2, attn_scales=(), temporal_downsample=(False, True, True)):
        super().__init__()
        self.variant = variant
        t_up = tuple(temporal_downsample[::-1])
        if variant == "wan2.1":
            dim, z_dim = dim or 96, z_dim or 16
            self.encoder = Encoder3d(dim, z_dim * 2, dim_mult, num_res_blocks, attn_scales, temporal_downsample)
            self.decoder = Decoder3d(dim, z_dim, dim_mult, num_res_blocks, attn_scales, t_up)
        elif variant == "wan2.2":
            dim, z_dim, dec_dim = dim or 160, z_dim or 48, dec_dim or 256
            self.encoder = Encoder3d38(dim, z_dim * 2, dim_mult, num_res_blocks, temporal_downsample)
            self.decoder = Decoder3d38(dec_dim, z_dim, dim_mult, num_res_blocks, t_up)
        else:
            raise ValueError(f"unknown autoencoder variant '{variant}' (wan2.1 | wan2.2)")
        self.z_dim = z_dim
        self.conv1 = CausalConv3d(z_dim * 2, z_dim * 2, 1)
        self.conv2 = CausalConv3d(z_dim, z_dim, 1)

    def encode(self, x, mean, inv_std):
        if self.variant == "wan2.2":
            x = fold2x2(x)
        mu, _ = self.conv1(self.encoder(x)).chunk(2, 1)
        return (mu - mean.view(1, -1, 1, 1, 1).to(mu)) * inv_std.view(1, -1, 1, 1, 1).to(mu)

    def decode(self, z, mean, inv_std):
        z = z / inv_std.view(1, -1, 1, 1, 1).to(z) + mean.view(1, -1, 1, 1, 1).to(z)
        out = self.decoder(self.conv2(z))
        return unfold2x2(out) if self.variant == "wan2.2" else out


class WanVAE(nn.Module):
    """Frozen autoencoder as the video model holds it: ``encode`` a list (or batch) of ``[3, T, H, W]`` videos in
    ``[-1, 1]`` with ``T = 1 + 4k`` into latents ``[z, 1 + k, H / s, W / s]``; ``decode`` back."""

    def __init__(self, variant: str = "wan2.1", mean: Optional[Sequence[float]] = None, std: Optional[Sequence[float]] = None, **kw):
        super().__init__()
        self.model = VideoVAE(variant, **kw).eval().requires_grad_(False)
        z = self.model.z_dim
        if mean is None or std is None:
            if variant == "wan2.1" and z == 16:
                mean, std = WAN21_MEAN, WAN21_STD
            else:  # released statistics travel in the model config (``vae_latent_mean`` / ``vae_latent_std``)
                mean, std = [0.0] * z, [1.0] * z
        self.register_buffer("mean", torch.tensor(list(mean), dtype=torch.float32), persistent=False)
        self.register_buffer("inv_std", 1.0 / torch.tensor(list(std), dtype=torch.float32), persistent=False)
        self.upsampling_factor = 8 if variant == "wan2.1" else 16
        self.z_dim = z

    @torch.no_grad()
    def encode(self, videos) -> torch.Tensor:
        if torch.is_tensor(videos) and videos.dim() == 5:
            return self.model.encode(videos.to(self.model.conv1.weight.dtype), self.mean, self.inv_std)
        return torch.stack([self.model.encode(v[None].to(self.model.conv1.weight.dtype), self.mean, self.inv_std)[0] for v in videos])

    @torch.no_grad()
    def decode(self, latents: torch.Tensor) -> torch.Tensor:
        if latents.dim() == 4:
            latents = latents[None]
        return self.model.decode(latents.to(self.model.conv2.weight.dtype), self.mean, self.inv_std).clamp_(-1, 1)
