"""Representation autoencoder on a SigLIP encoder (``model_type: rae_siglip``) with its perceptual and
adversarial critics.

* ``RaeSiglip``: frozen SigLIP vision encoder (last hidden state through an affine-free post-LayerNorm, optional
  per-sample noise of random strength and latent normalisation) and a trainable MAE-style ViT decoder
  (linear embed, trainable class token, fixed 2-D sin-cos positions, pre-LN blocks, linear pixel head,
  un-patchify and de-normalise).  Parameter names follow the reference's checkpoints
  (src/lmms_engine/models/rae_siglip/modeling_rae_siglip.py:31-202, general_decoder.py:290-472), so its
  ``encoder.*`` / ``decoder.*`` state dicts load directly.  Both towers run on the engine's packed kernels: every
  image is one document of the varlen attention kernel.
* ``Lpips``: VGG-16 perceptual distance with learned 1x1 heads (src/lmms_engine/models/rae_siglip/lpips.py:11-109).
  Weights come from files (``vgg_path``: torchvision's ``features.N`` layout, ``lin_path``: the published
  ``lin{k}.model.1.weight`` heads); nothing is downloaded.
* ``DinoDiscriminator``: frozen DINO ViT whose intermediate activations feed spectral-norm 1-D convolution heads
  (src/lmms_engine/models/rae_siglip/discriminator.py:197-381, 398-505); backbone keys are the timm layout of the
  published DINO checkpoints.
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
from .llava_ov import SiglipConfig, _VisionModel
from .vision import LayerNorm

SIGLIP_MEAN = (0.5, 0.5, 0.5)
SIGLIP_STD = (0.5, 0.5, 0.5)


# ------------------------------------------------------------------------------------ config
@dataclass
class MaeDecoderConfig:
    hidden_size: int = 768  # width of the latent that enters the decoder (set from the encoder)
    decoder_hidden_size: int = 512
    decoder_num_hidden_layers: int = 8
    decoder_num_attention_heads: int = 16
    decoder_intermediate_size: int = 2048
    patch_size: int = 16
    image_size: int = 224
    num_channels: int = 3
    layer_norm_eps: float = 1e-12
    hidden_act: str = "gelu"

    @classmethod
    def from_dict(cls, d):
        known = {f.name for f in fields(cls)}
        return cls(**{k: v for k, v in (d or {}).items() if k in known})


@dataclass
class RaeSiglipConfig:
    model_type: str = "rae_siglip"
    encoder_config: Any = None
    decoder_config: Any = None
    noise_tau: float = 0.8
    reshape_to_2d: bool = True
    latent_mean: Optional[List[float]] = None
    latent_var: Optional[List[float]] = None
    eps: float = 1e-5
    image_mean: Sequence[float] = SIGLIP_MEAN
    image_std: Sequence[float] = SIGLIP_STD
    extra: Dict[str, Any] = field(default_factory=dict)

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "RaeSiglipConfig":
        d = dict(d)
        enc, dec = dict(d.pop("encoder_config", None) or {}), dict(d.pop("decoder_config", None) or {})
        if not enc and "encoder_dim" in d:  # flat form: a small encoder / decoder described by a handful of sizes
            enc = dict(hidden_size=d.pop("encoder_dim"), num_hidden_layers=d.pop("encoder_depth", 12),
                       num_attention_heads=d.pop("encoder_heads", 12), image_size=d.get("image_size", 224),
                       patch_size=d.get("patch_size", 16))
            enc["intermediate_size"] = 4 * enc["hidden_size"]
            dec = dict(decoder_hidden_size=d.pop("decoder_dim", 512), decoder_num_hidden_layers=d.pop("decoder_depth", 8),
                       decoder_num_attention_heads=d.pop("decoder_heads", 8))
            dec["decoder_intermediate_size"] = 4 * dec["decoder_hidden_size"]
            d.pop("image_size", None), d.pop("patch_size", None)
        known = {f.name for f in fields(cls)}
        cfg = cls(**{k: v for k, v in d.items() if k in known and k not in ("encoder_config", "decoder_config", "extra")})
        cfg.extra = {k: v for k, v in d.items() if k not in known}
        cfg.encoder_config = SiglipConfig.from_dict(enc)
        # the decoder works on the encoder's grid: same patch size, same number of patches, latent width = encoder width
        dec.update(hidden_size=cfg.encoder_config.hidden_size, patch_size=cfg.encoder_config.patch_size,
                   image_size=cfg.encoder_config.image_size // cfg.encoder_config.patch_size * cfg.encoder_config.patch_size)
        cfg.decoder_config = MaeDecoderConfig.from_dict(dec)
        return cfg

    def to_dict(self):
        d = {f.name: getattr(self, f.name) for f in fields(self) if f.name not in ("encoder_config", "decoder_config", "extra")}
        d["image_mean"], d["image_std"] = list(self.image_mean), list(self.image_std)
        d["encoder_config"] = {"model_type": "siglip_vision_model", **{f.name: getattr(self.encoder_config, f.name) for f in fields(self.encoder_config)}}
        d["decoder_config"] = {"model_type": "vit_mae", **{f.name: getattr(self.decoder_config, f.name) for f in fields(self.decoder_config)}}
        d["architectures"] = ["RaeSiglipModel"]
        d.update(self.extra)
        return d


# ------------------------------------------------------------------------------------ decoder
def sincos_2d_with_cls(dim: int, side: int) -> torch.Tensor:
    """MAE's fixed table ``[1 + side^2, dim]``: first half of the channels encodes the column, second half the row
    (each half: sines then cosines); row 0 (class token) is zero."""
    def one(d, pos):
        omega = 1.0 / 10000 ** (np.arange(d // 2, dtype=np.float64) / (d / 2.0))
        out = np.einsum("m,d->md", pos.reshape(-1), omega)
        return np.concatenate([np.sin(out), np.cos(out)], 1)

    gh, gw = np.arange(side, dtype=np.float32), np.arange(side, dtype=np.float32)
    grid = np.stack(np.meshgrid(gw, gh), 0).reshape(2, 1, side, side)  # [0]: column index, [1]: row index
    emb = np.concatenate([one(dim // 2, grid[0]), one(dim // 2, grid[1])], 1)
    return torch.from_numpy(np.concatenate([np.zeros((1, dim)), emb], 0)).float()


class _Named(nn.Module):
    """A module whose only job is to give a child the name it has in the checkpoints."""

    def __init__(self, **children):
        super().__init__()
        for k, v in children.items():
            setattr(self, k, v)


class MaeLayer(nn.Module):
    def __init__(self, d: int, heads: int, inter: int, eps: float):
        super().__init__()
        self.heads, self.head_dim = heads, d // heads
        self.layernorm_before, self.layernorm_after = LayerNorm(d, eps), LayerNorm(d, eps)
        self.attention = _Named(attention=_Named(query=nn.Linear(d, d), key=nn.Linear(d, d), value=nn.Linear(d, d)),
                                output=_Named(dense=nn.Linear(d, d)))
        self.intermediate = _Named(dense=nn.Linear(d, inter))
        self.output = _Named(dense=nn.Linear(inter, d))

    def forward(self, x, cu):
        a = self.attention.attention
        P = x.shape[0]
        w = torch.cat([a.query.weight, a.key.weight, a.value.weight], 0)
        b = torch.cat([a.query.bias, a.key.bias, a.value.bias], 0)
        qkv = gemm_ops.linear(self.layernorm_before(x), w, b).view(P, 3, self.heads, self.head_dim)
        o = attn_ops.varlen_attn(qkv[:, 0], qkv[:, 1], qkv[:, 2], cu, cu, causal=False, softmax_scale=self.head_dim ** -0.5)
        x = x + gemm_ops.linear(o.reshape(P, -1), self.attention.output.dense.weight, self.attention.output.dense.bias)
        h = F.gelu(gemm_ops.linear(self.layernorm_after(x), self.intermediate.dense.weight, self.intermediate.dense.bias))
        return x + gemm_ops.linear(h, self.output.dense.weight, self.output.dense.bias)


class MaeDecoder(nn.Module):
    def __init__(self, c: MaeDecoderConfig, num_patches: int):
        super().__init__()
        self.config, self.num_patches = c, num_patches
        D = c.decoder_hidden_size
        self.decoder_embed = nn.Linear(c.hidden_size, D)
        side = int(math.isqrt(num_patches))
        self.decoder_pos_embed = nn.Parameter(sincos_2d_with_cls(D, side)[None], requires_grad=False)
        self.decoder_layers = nn.ModuleList([MaeLayer(D, c.decoder_num_attention_heads, c.decoder_intermediate_size, c.layer_norm_eps)
                                             for _ in range(c.decoder_num_hidden_layers)])
        self.decoder_norm = LayerNorm(D, c.layer_norm_eps)
        self.decoder_pred = nn.Linear(D, c.patch_size ** 2 * c.num_channels)
        self.trainable_cls_token = nn.Parameter(torch.zeros(1, 1, D))
        self.gradient_checkpointing = False

    def interpolate_latent(self, x):
        """Latents on another grid than the decoder's are resampled bilinearly."""
        b, l, c = x.shape
        if l == self.num_patches:
            return x
        h, t = int(math.isqrt(l)), int(math.isqrt(self.num_patches))
        x = F.interpolate(x.view(b, h, h, c).permute(0, 3, 1, 2).float(), size=(t, t), mode="bilinear", align_corners=False)
        return x.permute(0, 2, 3, 1).reshape(b, self.num_patches, c)

    def forward(self, latents: torch.Tensor):
        """``[B, N, hidden]`` -> ``(pixels per patch [B, N, p*p*C], last hidden state [B, N, D])``."""
        x = self.interpolate_latent(latents)
        B, N, _ = x.shape
        x = gemm_ops.linear(x.reshape(B * N, -1).to(self.decoder_embed.weight.dtype), self.decoder_embed.weight, self.decoder_embed.bias)
        x = torch.cat([self.trainable_cls_token.expand(B, -1, -1).to(x.dtype), x.view(B, N, -1)], 1)
        x = (x + self.decoder_pos_embed.to(x.dtype)).reshape(B * (N + 1), -1)
        cu = (torch.arange(B + 1, device=x.device) * (N + 1)).to(torch.int32)
        for layer in self.decoder_layers:
            if self.gradient_checkpointing and self.training:
                x = torch.utils.checkpoint.checkpoint(layer, x, cu, use_reentrant=False)
            else:
                x = layer(x, cu)
        h = self.decoder_norm(x)
        logits = gemm_ops.linear(h, self.decoder_pred.weight, self.decoder_pred.bias)
        self.last_layer_io = (h, logits) if logits.requires_grad else None
        return logits.view(B, N + 1, -1)[:, 1:], h.view(B, N + 1, -1)[:, 1:]

    def unpatchify(self, patches: torch.Tensor, size: Optional[Tuple[int, int]] = None) -> torch.Tensor:
        c = self.config
        H, W = size or (c.image_size, c.image_size)
        gh, gw, p = H // c.patch_size, W // c.patch_size, c.patch_size
        if gh * gw != patches.shape[1]:
            raise ValueError(f"{patches.shape[1]} patches do not tile a {H}x{W} image with patch {p}")
        x = patches.reshape(patches.shape[0], gh, gw, p, p, c.num_channels)
        return torch.einsum("nhwpqc->nchpwq", x).reshape(patches.shape[0], c.num_channels, gh * p, gw * p)


# ------------------------------------------------------------------------------------ autoencoder
class _PlainLayerNorm(nn.Module):
    """LayerNorm without scale and shift (the encoder's last norm carries no parameters in the checkpoints)."""

    def __init__(self, eps: float):
        super().__init__()
        self.eps = eps

    def forward(self, x):
        return F.layer_norm(x.float(), x.shape[-1:], None, None, self.eps).to(x.dtype)


class RaeSiglip(nn.Module):
    config_class = RaeSiglipConfig
    _no_split_modules = ["SiglipEncoderLayer", "MaeLayer"]

    def __init__(self, cfg: RaeSiglipConfig):
        super().__init__()
        self.config = cfg
        ec = cfg.encoder_config
        self.encoder_input_size, self.encoder_patch_size = ec.image_size, ec.patch_size
        self.base_patches = (ec.image_size // ec.patch_size) ** 2
        self.encoder = _VisionModel(ec)
        self.encoder.post_layernorm = _PlainLayerNorm(ec.layer_norm_eps)
        self.encoder.requires_grad_(False)
        self.decoder = MaeDecoder(cfg.decoder_config, self.base_patches)
        self.register_buffer("encoder_mean", torch.tensor(list(cfg.image_mean)).view(1, 3, 1, 1), persistent=False)
        self.register_buffer("encoder_std", torch.tensor(list(cfg.image_std)).view(1, 3, 1, 1), persistent=False)
        self.do_normalization = cfg.latent_mean is not None and cfg.latent_var is not None
        if self.do_normalization:
            self.register_buffer("latent_mean", torch.tensor(cfg.latent_mean, dtype=torch.float32), persistent=False)
            self.register_buffer("latent_var", torch.tensor(cfg.latent_var, dtype=torch.float32), persistent=False)
        self.discriminator: Optional[nn.Module] = None  # attached by the trainer (kept out of the autoencoder's checkpoint)
        for m in self.decoder.modules():
            if isinstance(m, nn.Linear):
                nn.init.xavier_uniform_(m.weight)
                nn.init.zeros_(m.bias)
        nn.init.normal_(self.decoder.trainable_cls_token, std=0.02)

    def last_layer(self) -> torch.Tensor:
        """Weight on which the adversarial term is balanced against the reconstruction term."""
        return self.decoder.decoder_pred.weight

    def last_layer_io(self):
        """Input rows and output of the last layer in the most recent training pass: the gradient of a loss with respect
        to the last layer's weight is ``d_output^T @ input``, whatever wrapper holds the weight itself in shards."""
        return getattr(self.decoder, "last_layer_io", None)

    def gradient_checkpointing_enable(self, **_):
        self.decoder.gradient_checkpointing = True

    # ---- halves -------------------------------------------------------------------------------------------
    @torch.no_grad()
    def encode(self, pixel_values: torch.Tensor) -> torch.Tensor:
        """Pixels in ``[0, 1]`` ``[B, 3, H, W]`` -> latent ``[B, hidden, side, side]`` (or ``[B, N, hidden]``)."""
        if pixel_values.dim() != 4:
            raise ValueError("pixel_values must be [batch, channels, height, width]")
        x = pixel_values.float()
        S = self.encoder_input_size
        if x.shape[-2] != S or x.shape[-1] != S:
            x = F.interpolate(x, size=(S, S), mode="bicubic", align_corners=False)
        x = (x - self.encoder_mean) / self.encoder_std
        vm = self.encoder
        B = x.shape[0]
        h = vm.embeddings(x.to(vm.embeddings.patch_embedding.weight.dtype))
        per = vm.embeddings.side ** 2
        cu = (torch.arange(B + 1, device=h.device) * per).to(torch.int32)
        for layer in vm.encoder.layers:
            h = layer(h, cu)
        h = vm.post_layernorm(h).view(B, per, -1)
        if self.training and self.config.noise_tau > 0:
            sigma = self.config.noise_tau * torch.rand((B, 1, 1), device=h.device, dtype=h.dtype)
            h = h + sigma * torch.randn_like(h)
        if self.config.reshape_to_2d:
            side = vm.embeddings.side
            h = h.transpose(1, 2).reshape(B, -1, side, side)
        if self.do_normalization:
            h = (h - self.latent_mean.to(h.dtype)) / torch.sqrt(self.latent_var.to(h.dtype) + self.config.eps)
        return h

    def decode(self, latent: torch.Tensor) -> Dict[str, torch.Tensor]:
        if latent.dim() == 3 and self.config.reshape_to_2d:
            B, N, D = latent.shape
            side = int(math.isqrt(N))
            if side * side != N:
                raise ValueError(f"{N} latent tokens do not form a square grid")
            latent = latent.transpose(1, 2).reshape(B, D, side, side)
        if latent.dim() not in (3, 4):
            raise ValueError("latent must be [batch, tokens, dim] or [batch, dim, h, w]")
        if self.do_normalization:
            latent = latent * torch.sqrt(self.latent_var.to(latent.dtype) + self.config.eps) + self.latent_mean.to(latent.dtype)
        if latent.dim() == 4:
            B, C, H, W = latent.shape
            latent = latent.reshape(B, C, H * W).transpose(1, 2)
        logits, hidden = self.decoder(latent)
        pixels = self.decoder.unpatchify(logits.float())
        return {"hidden_states": hidden, "out_pixels": pixels * self.encoder_std + self.encoder_mean}

    def forward(self, pixel_values=None, **_):
        out = self.decode(self.encode(pixel_values))
        target = pixel_values.float()
        if target.shape[-2:] != out["out_pixels"].shape[-2:]:
            target = F.interpolate(target, size=out["out_pixels"].shape[-2:], mode="bicubic", align_corners=False)
        out["loss"] = (out["out_pixels"] - target).abs().mean()
        out["reconstruction"] = out["out_pixels"]
        return out

    def convert_hf_state_dict(self, sd: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        """Reference checkpoints hold ``encoder.*`` (a SigLIP ``vision_model`` without the pooling head and without
        post-LayerNorm parameters) and ``decoder.*``; both layouts are this module's own."""
        return {k: v for k, v in sd.items() if not k.startswith("encoder.head.") and not k.startswith("discriminator.")}


# ------------------------------------------------------------------------------------ LPIPS
VGG16_LAYOUT = (64, 64, "M", 128, 128, "M", 256, 256, 256, "M", 512, 512, 512, "M", 512, 512, 512)
VGG16_TAPS = (3, 8, 15, 22, 29)  # indices (torchvision ``features`` numbering) of relu1_2 ... relu5_3


class Lpips(nn.Module):
    """Learned perceptual distance: unit-normalised VGG-16 activations at five depths, squared differences weighted by
    non-negative learned 1x1 heads, averaged over space and summed over depths.  Inputs in ``[-1, 1]``."""

    def __init__(self, vgg_path: Optional[str] = None, lin_path: Optional[str] = None, allow_random: bool = False):
        super().__init__()
        layers: List[nn.Module] = []
        c_in = 3
        for v in VGG16_LAYOUT:
            if v == "M":
                layers.append(nn.MaxPool2d(2, 2))
            else:
                layers += [nn.Conv2d(c_in, v, 3, padding=1), nn.ReLU(inplace=False)]
                c_in = v
        self.features = nn.Sequential(*layers)
        self.chns = (64, 128, 256, 512, 512)
        self.lins = nn.ModuleList([nn.Conv2d(c, 1, 1, bias=False) for c in self.chns])
        self.register_buffer("shift", torch.tensor([-0.030, -0.088, -0.188]).view(1, 3, 1, 1), persistent=False)
        self.register_buffer("scale", torch.tensor([0.458, 0.448, 0.450]).view(1, 3, 1, 1), persistent=False)
        if vgg_path:
            sd = torch.load(vgg_path, map_location="cpu")
            sd = {k[len("features."):]: v for k, v in sd.items() if k.startswith("features.")}
            self.features.load_state_dict(sd)
        if lin_path:
            sd = torch.load(lin_path, map_location="cpu")
            for i, lin in enumerate(self.lins):
                lin.weight.data.copy_(sd[f"lin{i}.model.1.weight"])
        if not (vgg_path and lin_path) and not allow_random:
            raise FileNotFoundError(
                "the perceptual loss needs pretrained weights: gan_config.lpips_vgg_path (torchvision VGG-16 state dict) and "
                "gan_config.lpips_lin_path (LPIPS linear heads); set perceptual_weight: 0 to train without it")
        self.requires_grad_(False)
        self.eval()

    def taps(self, x: torch.Tensor) -> List[torch.Tensor]:
        out = []
        for i, layer in enumerate(self.features):
            x = layer(x)
            if i in VGG16_TAPS:
                out.append(x)
        return out

    def forward(self, a: torch.Tensor, b: torch.Tensor, reduction: str = "mean") -> torch.Tensor:
        fa, fb = self.taps((a - self.shift) / self.scale), self.taps((b - self.shift) / self.scale)
        total = 0.0
        for lin, x, y in zip(self.lins, fa, fb):
            x = x / (x.pow(2).sum(1, keepdim=True).sqrt() + 1e-10)
            y = y / (y.pow(2).sum(1, keepdim=True).sqrt() + 1e-10)
            total = total + lin((x - y) ** 2).mean((2, 3), keepdim=True)
        if reduction == "none":
            return total
        return total.sum() if reduction == "sum" else total.mean()


# ------------------------------------------------------------------------------------ DINO discriminator
DINO_RECIPES = {
    "S_16": dict(depth=12, patch_size=16, embed_dim=384, num_heads=6, mlp_ratio=4.0),
    "S_8": dict(depth=12, patch_size=8, embed_dim=384, num_heads=6, mlp_ratio=4.0),
    "B_16": dict(depth=12, patch_size=16, embed_dim=768, num_heads=12, mlp_ratio=4.0),
}


class _DinoBlock(nn.Module):
    def __init__(self, d, heads, ratio, eps):
        super().__init__()
        self.heads, self.head_dim = heads, d // heads
        self.norm1, self.norm2 = LayerNorm(d, eps), LayerNorm(d, eps)
        self.attn = _Named(qkv=nn.Linear(d, 3 * d), proj=nn.Linear(d, d))
        self.mlp = _Named(fc1=nn.Linear(d, int(d * ratio)), fc2=nn.Linear(int(d * ratio), d))

    def forward(self, x, cu):
        P = x.shape[0]
        qkv = gemm_ops.linear(self.norm1(x), self.attn.qkv.weight, self.attn.qkv.bias).view(P, 3, self.heads, self.head_dim)
        o = attn_ops.varlen_attn(qkv[:, 0], qkv[:, 1], qkv[:, 2], cu, cu, causal=False, softmax_scale=self.head_dim ** -0.5)
        x = x + gemm_ops.linear(o.reshape(P, -1), self.attn.proj.weight, self.attn.proj.bias)
        h = F.gelu(gemm_ops.linear(self.norm2(x), self.mlp.fc1.weight, self.mlp.fc1.bias), approximate="tanh")
        return x + gemm_ops.linear(h, self.mlp.fc2.weight, self.mlp.fc2.bias)


class FrozenDino(nn.Module):
    """DINO ViT used as a fixed feature space.  ``forward`` takes images in ``[-1, 1]``, resizes them to 224, applies the
    ImageNet statistics and returns the patch activations ``[B, C, N]`` of the last block followed by those after each
    block in ``key_depths``."""

    def __init__(self, depth=12, key_depths=(2, 5, 8, 11), norm_eps=1e-6, patch_size=16, embed_dim=384, num_heads=6, mlp_ratio=4.0,
                 img_size: int = 224):
        super().__init__()
        self.embed_dim, self.patch_size, self.img_size = embed_dim, patch_size, img_size
        self.side = img_size // patch_size
        self.patch_embed = _Named(proj=nn.Conv2d(3, embed_dim, patch_size, patch_size))
        self.cls_token = nn.Parameter(torch.zeros(1, 1, embed_dim))
        self.pos_embed = nn.Parameter(torch.zeros(1, self.side ** 2 + 1, embed_dim))
        self.key_depths = tuple(sorted(d for d in key_depths if d < depth))
        self.blocks = nn.ModuleList([_DinoBlock(embed_dim, num_heads, mlp_ratio, norm_eps) for _ in range(depth)])
        self.norm = LayerNorm(embed_dim, norm_eps)  # in the checkpoints; the discriminator taps the blocks before it
        mean, std = torch.tensor((0.485, 0.456, 0.406)), torch.tensor((0.229, 0.224, 0.225))
        self.register_buffer("x_scale", (0.5 / std).view(1, 3, 1, 1), persistent=False)
        self.register_buffer("x_shift", ((0.5 - mean) / std).view(1, 3, 1, 1), persistent=False)
        self.requires_grad_(False)
        self.eval()

    def load_dino(self, sd: Dict[str, torch.Tensor]):
        sd = dict(sd)
        for k, v in sd.items():  # the key bias does not change a softmax over keys; the published recipe zeroes it
            if k.endswith(".attn.qkv.bias"):
                v = v.clone()
                C = v.numel() // 3
                v[C:2 * C] = 0
                sd[k] = v
        missing, unexpected = self.load_state_dict(sd, strict=False)
        if missing or unexpected:
            raise RuntimeError(f"DINO checkpoint does not match: missing {missing[:4]}, unexpected {unexpected[:4]}")

    def train(self, mode: bool = True):
        return super().train(False)  # stays in eval mode whatever its parent does

    def forward(self, x: torch.Tensor) -> List[torch.Tensor]:
        if x.shape[-1] != self.img_size or x.shape[-2] != self.img_size:
            x = F.interpolate(x, size=(self.img_size, self.img_size), mode="bilinear", align_corners=False)
        x = x * self.x_scale + self.x_shift
        B = x.shape[0]
        p, side = self.patch_size, self.side
        w = self.patch_embed.proj.weight
        rows = x.reshape(B, 3, side, p, side, p).permute(0, 2, 4, 1, 3, 5).reshape(B * side * side, 3 * p * p)
        tok = gemm_ops.linear(rows.to(w.dtype), w.view(w.shape[0], -1), self.patch_embed.proj.bias).view(B, side * side, -1)
        tok = torch.cat([self.cls_token.expand(B, -1, -1).to(tok.dtype), tok], 1) + self.pos_embed.to(tok.dtype)
        n = tok.shape[1]
        h = tok.reshape(B * n, -1)
        cu = (torch.arange(B + 1, device=h.device) * n).to(torch.int32)
        acts = []
        for i, blk in enumerate(self.blocks):
            h = blk(h, cu)
            if i in self.key_depths:
                acts.append(h.view(B, n, -1)[:, 1:].transpose(1, 2))
        acts.insert(0, h.view(B, n, -1)[:, 1:].transpose(1, 2))
        return acts


class BatchNormLocal(nn.Module):
    """Batch statistics over groups of ``virtual_bs`` samples (and the sequence), in fp32; no running averages, so
    training and evaluation behave alike."""

    def __init__(self, channels: int, virtual_bs: int = 1, eps: float = 1e-6):
        super().__init__()
        self.virtual_bs, self.eps = virtual_bs, eps
        self.weight, self.bias = nn.Parameter(torch.ones(channels)), nn.Parameter(torch.zeros(channels))

    def forward(self, x):  # [B, C, N]
        shape, dt = x.shape, x.dtype
        g = -(-shape[0] // self.virtual_bs)
        x = x.float().view(g, -1, shape[-2], shape[-1])
        x = (x - x.mean((1, 3), keepdim=True)) / torch.sqrt(x.var((1, 3), keepdim=True, unbiased=False) + self.eps)
        x = x * self.weight[None, :, None] + self.bias[None, :, None]
        return x.view(shape).to(dt)


def _conv1d(c_in, c_out, k, spectral: bool, circular: bool = True):
    conv = nn.Conv1d(c_in, c_out, k, padding=k // 2, padding_mode="circular" if (circular and k > 1) else "zeros")
    return nn.utils.spectral_norm(conv, n_power_iterations=1, eps=1e-12, dim=0) if spectral else conv


def _disc_block(c, k, norm_type, eps, spectral):
    norm = BatchNormLocal(c, eps=eps) if norm_type == "bn" else nn.GroupNorm(32, c, eps=eps)
    return nn.Sequential(_conv1d(c, c, k, spectral), norm, nn.LeakyReLU(0.2))


class _Residual(nn.Module):
    def __init__(self, fn):
        super().__init__()
        self.fn, self.ratio = fn, 1 / math.sqrt(2)

    def forward(self, x):
        return (self.fn(x) + x) * self.ratio


class DinoDiscriminator(nn.Module):
    """Logits ``[B, (1 + len(key_depths)) * N]``: one head per tapped depth, every head a 1x1 block, a residual block of
    width ``ks`` over the (circularly padded) patch sequence and a 1x1 read-out.  Only the heads train."""

    def __init__(self, dino_ckpt_path: Optional[str] = None, ks: int = 9, key_depths=(2, 5, 8, 11), norm_type: str = "bn",
                 using_spec_norm: bool = True, norm_eps: float = 1e-6, recipe: str = "S_8", allow_random: bool = False,
                 backbone: Optional[Dict[str, Any]] = None):
        super().__init__()
        spec = dict(DINO_RECIPES[recipe]) if backbone is None else dict(backbone)
        self.dino = FrozenDino(key_depths=key_depths, norm_eps=norm_eps, **spec)
        if dino_ckpt_path:
            self.dino.load_dino(torch.load(dino_ckpt_path, map_location="cpu"))
        elif not allow_random:
            raise FileNotFoundError("the DINO discriminator needs gan_config.dino_ckpt_path (a timm-layout DINO ViT state dict)")
        else:
            nn.init.normal_(self.dino.pos_embed, std=0.02)
        C = self.dino.embed_dim
        self.heads = nn.ModuleList([
            nn.Sequential(_disc_block(C, 1, norm_type, norm_eps, using_spec_norm),
                          _Residual(_disc_block(C, ks, norm_type, norm_eps, using_spec_norm)),
                          _conv1d(C, 1, 1, using_spec_norm))
            for _ in range(len(self.dino.key_depths) + 1)])

    def forward(self, x_pm1: torch.Tensor) -> torch.Tensor:
        acts = self.dino(x_pm1)
        B = x_pm1.shape[0]
        return torch.cat([head(a.float()).view(B, -1) for head, a in zip(self.heads, acts)], 1)
