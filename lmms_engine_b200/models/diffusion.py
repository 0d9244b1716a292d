"""Generative (diffusion / flow) model families with native blocks:

* ``SiT``  - scalable interpolant transformer (class-conditional DiT blocks with adaLN-zero) and
  its ``Transport`` (linear / VP / GVP interpolant paths, velocity / noise / score prediction,
  Euler ODE and Euler-Maruyama SDE samplers).  Reference: src/lmms_engine/models/sit/models.py,
  src/lmms_engine/models/sit/transport/{path,transport,integrators}.py.
* ``WanDiT`` - video diffusion transformer (3-D patch embedding, 3-D rotary positions, self
  attention, text cross attention, timestep modulation) with ``FlowMatchScheduler``.
  Reference: src/lmms_engine/models/wanvideo/wan_video_dit.py:186-235,
  src/lmms_engine/models/wanvideo/wan_video_scheduler.py.
* ``RaeAutoencoder`` - frozen ViT encoder + ViT decoder and a patch discriminator for the
  representation-autoencoder GAN recipe.  Reference: src/lmms_engine/models/rae_siglip/.

Attention runs on the non-causal varlen kernel (one "document" per sample); everything else
uses the shared GEMM / norm operators, so these families inherit the same kernels as the LLMs.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field, fields
from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import attention as attn_ops
from ..ops import gemm as gemm_ops
from ..ops import rope as rope_ops


def _cfg_from(cls, d):
    known = {f.name for f in fields(cls)}
    return cls(**{k: v for k, v in d.items() if k in known})


def timestep_embedding(t: torch.Tensor, dim: int, max_period: float = 10000.0) -> torch.Tensor:
    half = dim // 2
    freqs = torch.exp(-math.log(max_period) * torch.arange(half, device=t.device, dtype=torch.float32) / half)
    args = t.float()[:, None] * freqs[None]
    return torch.cat([args.cos(), args.sin()], -1)


def sincos_2d(dim: int, h: int, w: int, device=None) -> torch.Tensor:
    def one(n, d):
        omega = 1.0 / (10000 ** (torch.arange(d // 2, dtype=torch.float32, device=device) / (d // 2)))
        out = torch.arange(n, dtype=torch.float32, device=device)[:, None] * omega[None]
        return torch.cat([out.sin(), out.cos()], -1)

    eh, ew = one(h, dim // 2), one(w, dim // 2)
    return torch.cat([eh[:, None].expand(h, w, -1), ew[None].expand(h, w, -1)], -1).reshape(h * w, dim)


class SelfAttention(nn.Module):
    def __init__(self, dim: int, heads: int, qk_norm: bool = False):
        super().__init__()
        self.heads, self.hd = heads, dim // heads
        self.qkv = nn.Linear(dim, 3 * dim)
        self.proj = nn.Linear(dim, dim)
        self.qk_norm = qk_norm
        if qk_norm:
            self.q_norm = nn.LayerNorm(self.hd, eps=1e-6)
            self.k_norm = nn.LayerNorm(self.hd, eps=1e-6)

    def forward(self, x, cu, cos=None, sin=None):
        T = x.shape[0]
        qkv = gemm_ops.linear(x, self.qkv.weight, self.qkv.bias).view(T, 3, self.heads, self.hd)
        q, k, v = qkv[:, 0], qkv[:, 1], qkv[:, 2]
        if self.qk_norm:
            q, k = self.q_norm(q), self.k_norm(k)
        if cos is not None:
            q, k = rope_ops.rope_apply(q, cos, sin), rope_ops.rope_apply(k, cos, sin)
        o = attn_ops.varlen_attn(q, k, v, cu, cu, causal=False)
        return gemm_ops.linear(o.reshape(T, -1), self.proj.weight, self.proj.bias)


class CrossAttention(nn.Module):
    def __init__(self, dim: int, heads: int, ctx_dim: int):
        super().__init__()
        self.heads, self.hd = heads, dim // heads
        self.q = nn.Linear(dim, dim)
        self.kv = nn.Linear(ctx_dim, 2 * dim)
        self.proj = nn.Linear(dim, dim)

    def forward(self, x, cu_x, ctx, cu_ctx):
        q = gemm_ops.linear(x, self.q.weight, self.q.bias).view(x.shape[0], self.heads, self.hd)
        kv = gemm_ops.linear(ctx, self.kv.weight, self.kv.bias).view(ctx.shape[0], 2, self.heads, self.hd)
        o = attn_ops.varlen_attn(q, kv[:, 0], kv[:, 1], cu_x, cu_ctx, causal=False)
        return gemm_ops.linear(o.reshape(x.shape[0], -1), self.proj.weight, self.proj.bias)


class Mlp(nn.Module):
    def __init__(self, dim: int, hidden: int):
        super().__init__()
        self.fc1, self.fc2 = nn.Linear(dim, hidden), nn.Linear(hidden, dim)

    def forward(self, x):
        return gemm_ops.linear(F.gelu(gemm_ops.linear(x, self.fc1.weight, self.fc1.bias), approximate="tanh"),
                               self.fc2.weight, self.fc2.bias)


def modulate(x, shift, scale):
    return x * (1 + scale) + shift


class DiTBlock(nn.Module):
    """adaLN-zero transformer block; optional text cross-attention."""

    def __init__(self, dim: int, heads: int, mlp_ratio: float = 4.0, ctx_dim: Optional[int] = None, qk_norm: bool = False):
        super().__init__()
        self.norm1 = nn.LayerNorm(dim, elementwise_affine=False, eps=1e-6)
        self.attn = SelfAttention(dim, heads, qk_norm)
        self.norm2 = nn.LayerNorm(dim, elementwise_affine=False, eps=1e-6)
        self.mlp = Mlp(dim, int(dim * mlp_ratio))
        self.cross = CrossAttention(dim, heads, ctx_dim) if ctx_dim else None
        self.norm3 = nn.LayerNorm(dim, eps=1e-6) if ctx_dim else None
        self.adaLN = nn.Linear(dim, 6 * dim)
        nn.init.zeros_(self.adaLN.weight)
        nn.init.zeros_(self.adaLN.bias)

    def forward(self, x, c_tok, cu, cos=None, sin=None, ctx=None, cu_ctx=None):
        """``c_tok``: conditioning vector broadcast per token ``[T, dim]``."""
        s1, g1, b1, s2, g2, b2 = F.linear(F.silu(c_tok), self.adaLN.weight, self.adaLN.bias).chunk(6, -1)
        x = x + b1 * self.attn(modulate(self.norm1(x), s1, g1), cu, cos, sin)
        if self.cross is not None and ctx is not None:
            x = x + self.cross(self.norm3(x), cu, ctx, cu_ctx)
        return x + b2 * self.mlp(modulate(self.norm2(x), s2, g2))


def _sample_cu(B: int, n: int, device) -> torch.Tensor:
    return torch.arange(0, (B + 1) * n, n, dtype=torch.int32, device=device)


# ------------------------------------------------------------------------------------ SiT
@dataclass
class SiTConfig:
    model_type: str = "sit"
    input_size: int = 32
    patch_size: int = 2
    in_channels: int = 4
    hidden_size: int = 1152
    depth: int = 28
    num_heads: int = 16
    mlp_ratio: float = 4.0
    num_classes: int = 1000
    class_dropout_prob: float = 0.1
    learn_sigma: bool = False
    path_type: str = "linear"
    prediction: str = "velocity"

    from_dict = classmethod(_cfg_from)

    def to_dict(self):
        return {f.name: getattr(self, f.name) for f in fields(self)}


class SiT(nn.Module):
    config_class = SiTConfig
    _no_split_modules = ["DiTBlock"]

    def __init__(self, cfg: SiTConfig):
        super().__init__()
        self.config = cfg
        p, C, D = cfg.patch_size, cfg.in_channels, cfg.hidden_size
        self.out_channels = C * 2 if cfg.learn_sigma else C
        self.x_embedder = nn.Linear(C * p * p, D)
        self.t_embedder = nn.Sequential(nn.Linear(256, D), nn.SiLU(), nn.Linear(D, D))
        self.y_embedder = nn.Embedding(cfg.num_classes + 1, D)
        self.blocks = nn.ModuleList([DiTBlock(D, cfg.num_heads, cfg.mlp_ratio) for _ in range(cfg.depth)])
        self.final_norm = nn.LayerNorm(D, elementwise_affine=False, eps=1e-6)
        self.final_ada = nn.Linear(D, 2 * D)
        self.final = nn.Linear(D, p * p * self.out_channels)
        for m in (self.final_ada, self.final):
            nn.init.zeros_(m.weight)
            nn.init.zeros_(m.bias)
        self.transport = Transport(cfg.path_type, cfg.prediction)

    def patchify(self, x):
        B, C, H, W = x.shape
        p = self.config.patch_size
        x = x.view(B, C, H // p, p, W // p, p).permute(0, 2, 4, 1, 3, 5)
        return x.reshape(B * (H // p) * (W // p), C * p * p), (H // p, W // p)

    def unpatchify(self, tok, B, hw):
        h, w = hw
        p, C = self.config.patch_size, self.out_channels
        return tok.view(B, h, w, C, p, p).permute(0, 3, 1, 4, 2, 5).reshape(B, C, h * p, w * p)

    def denoise(self, x, t, y):
        B = x.shape[0]
        tok, hw = self.patchify(x)
        n = hw[0] * hw[1]
        h = self.x_embedder(tok.to(self.x_embedder.weight.dtype))
        h = h + sincos_2d(h.shape[-1], hw[0], hw[1], h.device).to(h.dtype).repeat(B, 1)
        c = self.t_embedder(timestep_embedding(t, 256).to(h.dtype)) + self.y_embedder(y)
        c_tok = c.repeat_interleave(n, 0)
        cu = _sample_cu(B, n, x.device)
        for blk in self.blocks:
            h = blk(h, c_tok, cu)
        shift, scale = self.final_ada(F.silu(c_tok)).chunk(2, -1)
        out = self.final(modulate(self.final_norm(h), shift, scale))
        return self.unpatchify(out.float(), B, hw)[:, : self.config.in_channels]

    def forward(self, pixel_values=None, labels=None, x=None, y=None, **kw) -> Dict[str, Any]:
        x = pixel_values if x is None else x
        y = labels if y is None else y
        if self.training and self.config.class_dropout_prob > 0:
            drop = torch.rand(y.shape[0], device=y.device) < self.config.class_dropout_prob
            y = torch.where(drop, torch.full_like(y, self.config.num_classes), y)
        loss = self.transport.training_loss(lambda xt, t: self.denoise(xt, t, y), x.float())
        return {"loss": loss}


class Transport:
    """Interpolant ``x_t = alpha(t) x_1 + sigma(t) x_0`` between noise ``x_0`` and data ``x_1``."""

    def __init__(self, path_type: str = "linear", prediction: str = "velocity", eps: float = 1e-5):
        self.path, self.prediction, self.eps = path_type.lower(), prediction, eps

    def coefficients(self, t):
        if self.path == "linear":
            return t, 1 - t, torch.ones_like(t), -torch.ones_like(t)
        if self.path == "gvp":
            a, s = torch.sin(math.pi / 2 * t), torch.cos(math.pi / 2 * t)
            return a, s, math.pi / 2 * s, -math.pi / 2 * a
        if self.path == "vp":
            lo, hi = 0.1, 20.0
            lmc = -0.25 * (1 - t) ** 2 * (hi - lo) - 0.5 * (1 - t) * lo
            a = torch.exp(lmc)
            da = a * (0.5 * (1 - t) * (hi - lo) + 0.5 * lo)
            s = torch.sqrt((1 - a * a).clamp(min=1e-8))
            return a, s, da, -a * da / s
        raise ValueError(self.path)

    def training_loss(self, model, x1: torch.Tensor) -> torch.Tensor:
        B = x1.shape[0]
        t = torch.rand(B, device=x1.device) * (1 - 2 * self.eps) + self.eps
        x0 = torch.randn_like(x1)
        a, s, da, ds = (c.view(B, *([1] * (x1.dim() - 1))) for c in self.coefficients(t))
        xt = a * x1 + s * x0
        out = model(xt, t)
        if self.prediction == "velocity":
            target = da * x1 + ds * x0
        elif self.prediction == "noise":
            target = x0
        else:  # score
            target = -x0 / s
        return ((out - target) ** 2).mean()

    @torch.no_grad()
    def sample_ode(self, model, x0: torch.Tensor, steps: int = 50) -> torch.Tensor:
        x = x0
        ts = torch.linspace(self.eps, 1 - self.eps, steps + 1, device=x0.device)
        for i in range(steps):
            t = ts[i].expand(x.shape[0])
            x = x + (ts[i + 1] - ts[i]) * model(x, t)
        return x

    @torch.no_grad()
    def sample_sde(self, model, x0: torch.Tensor, steps: int = 250, diffusion: float = 1.0) -> torch.Tensor:
        """Euler-Maruyama on the velocity model with the score recovered from the velocity."""
        x = x0
        ts = torch.linspace(self.eps, 1 - self.eps, steps + 1, device=x0.device)
        for i in range(steps):
            t = ts[i].expand(x.shape[0])
            dt = ts[i + 1] - ts[i]
            v = model(x, t)
            a, s, da, ds = (c.view(-1, *([1] * (x.dim() - 1))) for c in self.coefficients(t))
            score = (a * v - da * x) / (s * (da * s - a * ds)).clamp(min=1e-6) if self.prediction == "velocity" else 0.0
            w = diffusion * s
            x = x + (v + 0.5 * w * score) * dt + torch.sqrt(w.clamp(min=0) * dt) * torch.randn_like(x)
        return x


# ------------------------------------------------------------------------------------ Wan DiT
@dataclass
class WanConfig:
    model_type: str = "wanvideo"
    in_dim: int = 16
    out_dim: int = 16
    dim: int = 1536
    ffn_dim: int = 8960
    num_heads: int = 12
    num_layers: int = 30
    text_dim: int = 4096
    freq_dim: int = 256
    patch_size: Tuple[int, int, int] = (1, 2, 2)
    num_train_timesteps: int = 1000
    shift: float = 5.0
    camera_control: bool = False

    from_dict = classmethod(_cfg_from)

    def to_dict(self):
        d = {f.name: getattr(self, f.name) for f in fields(self)}
        d["patch_size"] = list(self.patch_size)
        return d


class FlowMatchScheduler:
    """Shifted flow-matching schedule: ``sigma' = shift*sigma / (1 + (shift-1)*sigma)``."""

    def __init__(self, num_train_timesteps: int = 1000, shift: float = 5.0):
        self.n, self.shift = num_train_timesteps, shift
        s = torch.linspace(1.0, 0.0, num_train_timesteps + 1)[:-1]
        self.sigmas = shift * s / (1 + (shift - 1) * s)
        self.timesteps = self.sigmas * num_train_timesteps
        x = self.timesteps
        y = torch.exp(-2 * ((x - num_train_timesteps / 2) / num_train_timesteps) ** 2)
        y = y - y.min()
        self.weights = y * (num_train_timesteps / y.sum())

    def add_noise(self, x, noise, idx):
        s = self.sigmas.to(x.device)[idx].view(-1, *([1] * (x.dim() - 1)))
        return (1 - s) * x + s * noise

    def training_target(self, x, noise):
        return noise - x

    def training_weight(self, idx, device):
        return self.weights.to(device)[idx]

    def step(self, v, idx, x):
        s = self.sigmas.to(x.device)
        nxt = s[idx + 1] if idx + 1 < len(s) else torch.zeros((), device=x.device)
        return x + v * (nxt - s[idx])


class WanDiT(nn.Module):
    config_class = WanConfig
    _no_split_modules = ["DiTBlock"]

    def __init__(self, cfg: WanConfig):
        super().__init__()
        self.config = cfg
        pt, ph, pw = cfg.patch_size
        self.patch_embedding = nn.Linear(cfg.in_dim * pt * ph * pw, cfg.dim)
        self.text_embedding = nn.Sequential(nn.Linear(cfg.text_dim, cfg.dim), nn.GELU(approximate="tanh"), nn.Linear(cfg.dim, cfg.dim))
        self.time_embedding = nn.Sequential(nn.Linear(cfg.freq_dim, cfg.dim), nn.SiLU(), nn.Linear(cfg.dim, cfg.dim))
        self.blocks = nn.ModuleList([DiTBlock(cfg.dim, cfg.num_heads, cfg.ffn_dim / cfg.dim, ctx_dim=cfg.dim, qk_norm=True)
                                     for _ in range(cfg.num_layers)])
        self.head_norm = nn.LayerNorm(cfg.dim, elementwise_affine=False, eps=1e-6)
        self.head_ada = nn.Linear(cfg.dim, 2 * cfg.dim)
        self.head = nn.Linear(cfg.dim, cfg.out_dim * pt * ph * pw)
        if cfg.camera_control:
            self.camera_adapter = nn.Sequential(nn.Linear(6 * 64 * pt, cfg.dim), nn.SiLU(), nn.Linear(cfg.dim, cfg.dim))
        self.scheduler = FlowMatchScheduler(cfg.num_train_timesteps, cfg.shift)
        self.hd = cfg.dim // cfg.num_heads

    def rope_3d(self, f, h, w, device):
        hd = self.hd
        d_t = hd - 2 * (hd // 3 // 2 * 2)
        d_h = d_w = hd // 3 // 2 * 2
        def ang(n, d):
            inv = 1.0 / (10000 ** (torch.arange(0, d, 2, device=device, dtype=torch.float32) / d))
            return torch.arange(n, device=device, dtype=torch.float32)[:, None] * inv[None]
        at, ah, aw = ang(f, d_t), ang(h, d_h), ang(w, d_w)
        a = torch.cat([at[:, None, None].expand(f, h, w, -1), ah[None, :, None].expand(f, h, w, -1),
                       aw[None, None].expand(f, h, w, -1)], -1).reshape(f * h * w, -1)
        a = torch.cat([a, a], -1)
        return a.cos(), a.sin()

    def denoise(self, x, t, context, plucker=None):
        """``x [B, C, F, H, W]`` latents, ``t [B]``, ``context [B, L, text_dim]``."""
        B, C, Fr, H, W = x.shape
        pt, ph, pw = self.config.patch_size
        f, h, w = Fr // pt, H // ph, W // pw
        tok = x.view(B, C, f, pt, h, ph, w, pw).permute(0, 2, 4, 6, 1, 3, 5, 7).reshape(B * f * h * w, -1)
        hdn = self.patch_embedding(tok.to(self.patch_embedding.weight.dtype))
        if plucker is not None and self.config.camera_control:
            hdn = hdn + self.camera_adapter(plucker.to(hdn.dtype))
        n = f * h * w
        ctx = self.text_embedding(context.reshape(-1, context.shape[-1]).to(hdn.dtype))
        c = self.time_embedding(timestep_embedding(t, self.config.freq_dim).to(hdn.dtype))
        c_tok = c.repeat_interleave(n, 0)
        cu, cu_ctx = _sample_cu(B, n, x.device), _sample_cu(B, context.shape[1], x.device)
        cos, sin = self.rope_3d(f, h, w, x.device)
        cos, sin = cos.repeat(B, 1), sin.repeat(B, 1)
        for blk in self.blocks:
            hdn = blk(hdn, c_tok, cu, cos, sin, ctx, cu_ctx)
        shift, scale = self.head_ada(F.silu(c_tok)).chunk(2, -1)
        out = self.head(modulate(self.head_norm(hdn), shift, scale)).float()
        Co = self.config.out_dim
        return out.view(B, f, h, w, Co, pt, ph, pw).permute(0, 4, 1, 5, 2, 6, 3, 7).reshape(B, Co, Fr, H, W)

    def forward(self, latents=None, context=None, plucker=None, **kw) -> Dict[str, Any]:
        """Flow-matching loss: random timestep, noised latents, MSE to (noise - x) x weight(t)."""
        B = latents.shape[0]
        idx = torch.randint(0, self.scheduler.n, (B,), device=latents.device)
        noise = torch.randn_like(latents.float())
        noisy = self.scheduler.add_noise(latents.float(), noise, idx.cpu())
        t = self.scheduler.timesteps.to(latents.device)[idx]
        pred = self.denoise(noisy, t, context, plucker)
        target = self.scheduler.training_target(latents.float(), noise)
        w = self.scheduler.training_weight(idx.cpu(), latents.device).view(B, 1, 1, 1, 1)
        return {"loss": (w * (pred - target) ** 2).mean()}


# ------------------------------------------------------------------------------------ RAE
@dataclass
class RaeConfig:
    model_type: str = "rae_siglip"
    image_size: int = 224
    patch_size: int = 16
    encoder_dim: int = 768
    encoder_depth: int = 12
    encoder_heads: int = 12
    decoder_dim: int = 512
    decoder_depth: int = 8
    decoder_heads: int = 8
    noise_tau: float = 0.0
    disc_dim: int = 256

    from_dict = classmethod(_cfg_from)

    def to_dict(self):
        return {f.name: getattr(self, f.name) for f in fields(self)}


class _ViT(nn.Module):
    def __init__(self, dim, depth, heads, in_dim):
        super().__init__()
        self.inp = nn.Linear(in_dim, dim)
        self.blocks = nn.ModuleList([DiTBlock(dim, heads) for _ in range(depth)])
        self.norm = nn.LayerNorm(dim, eps=1e-6)
        self.zero_c = None

    def forward(self, tok, B, hw):
        n = hw[0] * hw[1]
        h = self.inp(tok) + sincos_2d(self.inp.out_features, hw[0], hw[1], tok.device).to(tok.dtype).repeat(B, 1)
        c = torch.zeros_like(h)
        cu = _sample_cu(B, n, tok.device)
        for blk in self.blocks:
            h = blk(h, c, cu)
        return self.norm(h)


class PatchDiscriminator(nn.Module):
    def __init__(self, in_ch: int = 3, dim: int = 256):
        super().__init__()
        self.net = nn.Sequential(
            nn.Conv2d(in_ch, dim // 4, 4, 2, 1), nn.LeakyReLU(0.2), nn.Conv2d(dim // 4, dim // 2, 4, 2, 1),
            nn.GroupNorm(8, dim // 2), nn.LeakyReLU(0.2), nn.Conv2d(dim // 2, dim, 4, 2, 1), nn.GroupNorm(8, dim),
            nn.LeakyReLU(0.2), nn.Conv2d(dim, 1, 3, 1, 1))

    def forward(self, x):
        return self.net(x)


class RaeAutoencoder(nn.Module):
    config_class = RaeConfig
    _no_split_modules = ["DiTBlock"]

    def __init__(self, cfg: RaeConfig):
        super().__init__()
        self.config = cfg
        p = cfg.patch_size
        self.encoder = _ViT(cfg.encoder_dim, cfg.encoder_depth, cfg.encoder_heads, 3 * p * p)
        self.decoder = _ViT(cfg.decoder_dim, cfg.decoder_depth, cfg.decoder_heads, cfg.encoder_dim)
        self.to_pixels = nn.Linear(cfg.decoder_dim, 3 * p * p)
        self.discriminator = PatchDiscriminator(3, cfg.disc_dim)
        for q in self.encoder.parameters():
            q.requires_grad_(False)

    def last_layer(self):
        return self.to_pixels.weight

    def last_layer_io(self):
        return getattr(self, "_last_io", None)

    def patchify(self, x):
        B, C, H, W = x.shape
        p = self.config.patch_size
        return x.view(B, C, H // p, p, W // p, p).permute(0, 2, 4, 1, 3, 5).reshape(-1, C * p * p), (H // p, W // p)

    def encode(self, x):
        tok, hw = self.patchify(x)
        with torch.no_grad():
            z = self.encoder(tok.to(self.encoder.inp.weight.dtype), x.shape[0], hw)
        if self.training and self.config.noise_tau > 0:
            z = z + self.config.noise_tau * torch.rand(()) * torch.randn_like(z)
        return z, hw

    def decode(self, z, B, hw):
        p = self.config.patch_size
        h = self.decoder(z, B, hw)
        out = self.to_pixels(h)
        self._last_io = (h, out) if out.requires_grad else None
        out = out.float()
        return out.view(B, hw[0], hw[1], 3, p, p).permute(0, 3, 1, 4, 2, 5).reshape(B, 3, hw[0] * p, hw[1] * p)

    def forward(self, pixel_values=None, **kw):
        z, hw = self.encode(pixel_values)
        rec = self.decode(z, pixel_values.shape[0], hw)
        return {"loss": (rec - pixel_values.float()).abs().mean(), "reconstruction": rec}
