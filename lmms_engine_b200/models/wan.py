"""Wan video diffusion family (``model_type: wanvideo``): the diffusion transformer in the released checkpoint layout,
the VACE hint branch, and the conditional-generation wrapper that owns the frozen autoencoder / text / image encoders.

Reference: src/lmms_engine/models/wanvideo/wan_video_dit.py:97-480 (blocks, head, patch / text / time embeddings),
wan_video_vace.py:7-100, modeling_wanvideo.py:48-672 (wrapper: freezing, prompt / video / image embedding,
denoising forward), src/lmms_engine/train/hf/wan_trainer.py:30-96 (flow-matching loss).

B200 mapping: all samples of a batch are packed into one token stream (``cu_seqlens`` per sample), so self- and
cross-attention run on the varlen tcgen05 kernel and every projection is one GEMM over the whole batch; q/k/v share one
GEMM.  The released rotary embedding rotates INTERLEAVED pairs with complex arithmetic; here q and k are
de-interleaved (a fixed permutation of the head dimension, which leaves every q.k product unchanged) so the
engine's half-split rotary kernel applies, with the 3-D angle table laid out to match.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field, fields
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import attention as attn_ops
from ..ops import gemm as gemm_ops
from ..ops import norm as norm_ops
from ..ops import rope as rope_ops
from .diffusion import FlowMatchScheduler
from .wan_encoders import WanImageEncoder, WanMotionController, WanTextEncoder, sinusoid_1d
from .wan_vae import WanVAE

_ALIASES = {"dim": "dit_hidden_size", "ffn_dim": "dit_intermediate_size", "num_heads": "dit_num_heads", "num_layers": "dit_num_layers",
            "text_dim": "dit_text_dim", "in_dim": "dit_in_channels", "out_dim": "dit_out_channels", "freq_dim": "dit_freq_dim",
            "patch_size": "dit_patch_size"}


@dataclass
class WanVideoConfig:
    model_type: str = "wanvideo"
    dit_hidden_size: int = 3072
    dit_num_layers: int = 30
    dit_num_heads: int = 24
    dit_intermediate_size: int = 14336
    dit_patch_size: Tuple[int, int, int] = (1, 2, 2)
    dit_in_channels: int = 48
    dit_out_channels: int = 48
    dit_freq_dim: int = 256
    dit_text_dim: int = 4096
    dit_eps: float = 1e-6
    dit_has_image_input: bool = False
    dit_has_image_pos_emb: bool = False
    dit_has_ref_conv: bool = False
    dit_add_control_adapter: bool = False
    dit_in_channels_control_adapter: int = 24
    trainable_modules: Optional[str] = "dit"
    seperated_timestep: bool = True
    require_clip_embedding: bool = False
    require_vae_embedding: bool = False
    fuse_vae_embedding_in_latents: bool = True
    # frozen towers; ``None`` leaves a tower out (training on stored latents / prompt embeddings)
    vae: Optional[Dict[str, Any]] = None  # e.g. {"variant": "wan2.2"}
    text_encoder: Optional[Dict[str, Any]] = None  # kwargs of WanTextEncoder ({} = umt5-xxl sizes)
    image_encoder: Optional[Dict[str, Any]] = None  # kwargs of ClipVisionTower ({} = ViT-H/14)
    motion_controller: bool = False
    vace: Optional[Dict[str, Any]] = None  # {"vace_layers": [...], "vace_in_dim": 96}
    num_train_timesteps: int = 1000
    shift: float = 5.0
    clip_dim: int = 1280
    clip_tokens: int = 257
    extra: Dict[str, Any] = field(default_factory=dict)

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "WanVideoConfig":
        d = {_ALIASES.get(k, k): v for k, v in dict(d).items()}
        known = {f.name for f in fields(cls)}
        cfg = cls(**{k: v for k, v in d.items() if k in known and k != "extra"})
        cfg.extra = {k: v for k, v in d.items() if k not in known}
        cfg.dit_patch_size = tuple(cfg.dit_patch_size)
        return cfg

    def to_dict(self):
        d = {f.name: getattr(self, f.name) for f in fields(self) if f.name != "extra"}
        d["dit_patch_size"] = list(self.dit_patch_size)
        d["architectures"] = ["WanVideoForConditionalGeneration"]
        d.update(self.extra)
        return d


# ------------------------------------------------------------------------------------ pieces
class WanRMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-5):
        super().__init__()
        self.weight, self.eps = nn.Parameter(torch.ones(dim)), eps

    def forward(self, x):
        return norm_ops.rmsnorm(x, self.weight, self.eps)


def rope_axes(head_dim: int) -> Tuple[int, int, int]:
    """Rotary PAIRS per axis (frame, row, column): ``d - 2 (d // 3)`` of the head dimension turn with the frame index,
    ``d // 3`` each with row and column."""
    hw = head_dim // 3
    return (head_dim - 2 * hw) // 2, hw // 2, hw // 2


def rope_table_3d(head_dim: int, f: int, h: int, w: int, device, theta: float = 10000.0, offset_f: int = 0):
    """Half-split cos / sin tables ``[f*h*w, head_dim]`` for de-interleaved q / k."""
    def ang(n, pairs, start=0):
        d = 2 * pairs
        inv = 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float64, device=device)[:pairs] / d))
        return torch.outer(torch.arange(start, start + n, dtype=torch.float64, device=device), inv)

    pf, ph, pw = rope_axes(head_dim)
    a = torch.cat([ang(f, pf, offset_f)[:, None, None].expand(f, h, w, -1), ang(h, ph)[None, :, None].expand(f, h, w, -1),
                   ang(w, pw)[None, None].expand(f, h, w, -1)], -1).reshape(f * h * w, -1)
    a = torch.cat([a, a], -1)
    return a.cos().float(), a.sin().float()


def _deinterleave(x):  # [T, H, D]: (re0, im0, re1, im1, ...) -> (re0, re1, ..., im0, im1, ...)
    T, H, D = x.shape
    return x.view(T, H, D // 2, 2).transpose(-1, -2).reshape(T, H, D)


class WanSelfAttention(nn.Module):
    def __init__(self, dim: int, heads: int, eps: float):
        super().__init__()
        self.heads, self.head_dim = heads, dim // heads
        self.q, self.k, self.v, self.o = (nn.Linear(dim, dim) for _ in range(4))
        self.norm_q, self.norm_k = WanRMSNorm(dim, eps), WanRMSNorm(dim, eps)

    def forward(self, x, cu, cos, sin):
        T, D = x.shape
        w = torch.cat([self.q.weight, self.k.weight, self.v.weight], 0)
        b = torch.cat([self.q.bias, self.k.bias, self.v.bias], 0)
        qkv = gemm_ops.linear(x, w, b)
        q = _deinterleave(self.norm_q(qkv[:, :D].contiguous()).view(T, self.heads, self.head_dim))
        k = _deinterleave(self.norm_k(qkv[:, D:2 * D].contiguous()).view(T, self.heads, self.head_dim))
        v = qkv[:, 2 * D:].view(T, self.heads, self.head_dim)
        q, k = rope_ops.rope_apply(q, cos, sin), rope_ops.rope_apply(k, cos, sin)
        o = attn_ops.varlen_attn(q, k, v, cu, cu, causal=False, softmax_scale=self.head_dim ** -0.5)
        return gemm_ops.linear(o.reshape(T, D), self.o.weight, self.o.bias)


class WanCrossAttention(nn.Module):
    def __init__(self, dim: int, heads: int, eps: float, has_image_input: bool):
        super().__init__()
        self.heads, self.head_dim = heads, dim // heads
        self.q, self.k, self.v, self.o = (nn.Linear(dim, dim) for _ in range(4))
        self.norm_q, self.norm_k = WanRMSNorm(dim, eps), WanRMSNorm(dim, eps)
        self.has_image_input = has_image_input
        if has_image_input:
            self.k_img, self.v_img = nn.Linear(dim, dim), nn.Linear(dim, dim)
            self.norm_k_img = WanRMSNorm(dim, eps)

    def _kv(self, ctx, k_lin, v_lin, norm):
        n = ctx.shape[0]
        kv = gemm_ops.linear(ctx, torch.cat([k_lin.weight, v_lin.weight], 0), torch.cat([k_lin.bias, v_lin.bias], 0))
        D = kv.shape[1] // 2
        return norm(kv[:, :D].contiguous()).view(n, self.heads, self.head_dim), kv[:, D:].view(n, self.heads, self.head_dim)

    def forward(self, x, cu, ctx, cu_ctx, img=None, cu_img=None):
        T, D = x.shape
        q = self.norm_q(gemm_ops.linear(x, self.q.weight, self.q.bias)).view(T, self.heads, self.head_dim)
        k, v = self._kv(ctx, self.k, self.v, self.norm_k)
        o = attn_ops.varlen_attn(q, k, v, cu, cu_ctx, causal=False, softmax_scale=self.head_dim ** -0.5)
        if self.has_image_input and img is not None:
            ki, vi = self._kv(img, self.k_img, self.v_img, self.norm_k_img)
            o = o + attn_ops.varlen_attn(q, ki, vi, cu, cu_img, causal=False, softmax_scale=self.head_dim ** -0.5)
        return gemm_ops.linear(o.reshape(T, D), self.o.weight, self.o.bias)


class WanDiTBlock(nn.Module):
    def __init__(self, has_image_input: bool, dim: int, heads: int, ffn_dim: int, eps: float = 1e-6):
        super().__init__()
        self.dim = dim
        self.self_attn = WanSelfAttention(dim, heads, eps)
        self.cross_attn = WanCrossAttention(dim, heads, eps, has_image_input)
        self.norm1 = nn.LayerNorm(dim, eps=eps, elementwise_affine=False)
        self.norm2 = nn.LayerNorm(dim, eps=eps, elementwise_affine=False)
        self.norm3 = nn.LayerNorm(dim, eps=eps)
        self.ffn = nn.Sequential(nn.Linear(dim, ffn_dim), nn.GELU(approximate="tanh"), nn.Linear(ffn_dim, dim))
        self.modulation = nn.Parameter(torch.randn(1, 6, dim) / dim ** 0.5)

    def forward(self, x, mod_tok, cu, cos, sin, ctx, cu_ctx, img=None, cu_img=None):
        """``mod_tok [T, 6, dim]``: the timestep modulation of every token's sample (or of the token itself)."""
        m = self.modulation.to(mod_tok.dtype) + mod_tok
        s1, c1, g1, s2, c2, g2 = m.unbind(1)
        x = x + g1 * self.self_attn(self.norm1(x) * (1 + c1) + s1, cu, cos, sin)
        x = x + self.cross_attn(self.norm3(x), cu, ctx, cu_ctx, img, cu_img)
        h = gemm_ops.linear(self.norm2(x) * (1 + c2) + s2, self.ffn[0].weight, self.ffn[0].bias)
        return x + g2 * gemm_ops.linear(F.gelu(h, approximate="tanh"), self.ffn[2].weight, self.ffn[2].bias)


class WanHead(nn.Module):
    def __init__(self, dim: int, out_channels: int, patch_size, eps: float):
        super().__init__()
        self.norm = nn.LayerNorm(dim, eps=eps, elementwise_affine=False)
        self.head = nn.Linear(dim, out_channels * math.prod(patch_size))
        self.modulation = nn.Parameter(torch.randn(1, 2, dim) / dim ** 0.5)

    def forward(self, x, t_tok):  # t_tok [T, dim]
        m = self.modulation.to(t_tok.dtype) + t_tok[:, None]
        return gemm_ops.linear(self.norm(x) * (1 + m[:, 1]) + m[:, 0], self.head.weight, self.head.bias)


class WanImageMLP(nn.Module):
    def __init__(self, in_dim: int, out_dim: int, has_pos_emb: bool = False, tokens: int = 514):
        super().__init__()
        self.proj = nn.Sequential(nn.LayerNorm(in_dim), nn.Linear(in_dim, in_dim), nn.GELU(), nn.Linear(in_dim, out_dim), nn.LayerNorm(out_dim))
        self.has_pos_emb = has_pos_emb
        if has_pos_emb:
            self.emb_pos = nn.Parameter(torch.zeros(1, tokens, in_dim))

    def forward(self, x):
        if self.has_pos_emb:
            x = x + self.emb_pos[:, : x.shape[1]].to(x.dtype)
        return self.proj(x)


class SimpleAdapter(nn.Module):
    """Camera-control adapter: pixel-unshuffle by 8, a strided convolution to the model width, one residual block."""

    def __init__(self, in_dim: int, out_dim: int, kernel_size, stride):
        super().__init__()
        self.pixel_unshuffle = nn.PixelUnshuffle(8)
        self.conv = nn.Conv2d(in_dim * 64, out_dim, kernel_size=kernel_size, stride=stride)
        self.residual_blocks = nn.Sequential(_AdapterBlock(out_dim))

    def forward(self, x):  # [B, C, F, H, W]
        b, c, f, h, w = x.shape
        y = self.residual_blocks(self.conv(self.pixel_unshuffle(x.permute(0, 2, 1, 3, 4).reshape(b * f, c, h, w))))
        return y.view(b, f, *y.shape[1:]).permute(0, 2, 1, 3, 4)


class _AdapterBlock(nn.Module):
    def __init__(self, dim):
        super().__init__()
        self.conv1, self.conv2 = nn.Conv2d(dim, dim, 3, padding=1), nn.Conv2d(dim, dim, 3, padding=1)

    def forward(self, x):
        return x + self.conv2(F.relu(self.conv1(x)))


class WanDit(nn.Module):
    def __init__(self, c: WanVideoConfig):
        super().__init__()
        D = c.dit_hidden_size
        self.config = c
        self.hidden_size, self.freq_dim, self.patch_size = D, c.dit_freq_dim, tuple(c.dit_patch_size)
        self.head_dim = D // c.dit_num_heads
        self.has_image_input = c.dit_has_image_input
        self.patch_embedding = nn.Conv3d(c.dit_in_channels, D, kernel_size=self.patch_size, stride=self.patch_size)
        self.text_embedding = nn.Sequential(nn.Linear(c.dit_text_dim, D), nn.GELU(approximate="tanh"), nn.Linear(D, D))
        self.time_embedding = nn.Sequential(nn.Linear(c.dit_freq_dim, D), nn.SiLU(), nn.Linear(D, D))
        self.time_projection = nn.Sequential(nn.SiLU(), nn.Linear(D, D * 6))
        self.blocks = nn.ModuleList([WanDiTBlock(c.dit_has_image_input, D, c.dit_num_heads, c.dit_intermediate_size, c.dit_eps)
                                     for _ in range(c.dit_num_layers)])
        self.head = WanHead(D, c.dit_out_channels, self.patch_size, c.dit_eps)
        if c.dit_has_image_input:
            self.img_emb = WanImageMLP(c.clip_dim, D, c.dit_has_image_pos_emb, 2 * c.clip_tokens)
        if c.dit_has_ref_conv:
            self.ref_conv = nn.Conv2d(c.dit_in_channels, D, kernel_size=(2, 2), stride=(2, 2))
        self.control_adapter = (SimpleAdapter(c.dit_in_channels_control_adapter, D, self.patch_size[1:], self.patch_size[1:])
                                if c.dit_add_control_adapter else None)
        self.gradient_checkpointing = False

    def patchify(self, x: torch.Tensor, camera: Optional[torch.Tensor] = None):
        """``[B, C, F, H, W]`` -> tokens ``[B, f*h*w, D]`` (the strided convolution as one GEMM) and the grid."""
        B, C, Fr, H, W = x.shape
        pt, ph, pw = self.patch_size
        f, h, w = Fr // pt, H // ph, W // pw
        rows = x.view(B, C, f, pt, h, ph, w, pw).permute(0, 2, 4, 6, 1, 3, 5, 7).reshape(B * f * h * w, C * pt * ph * pw)
        wgt = self.patch_embedding.weight
        tok = gemm_ops.linear(rows.to(wgt.dtype), wgt.view(wgt.shape[0], -1), self.patch_embedding.bias).view(B, f * h * w, -1)
        if self.control_adapter is not None and camera is not None:
            tok = tok + self.control_adapter(camera.to(wgt.dtype)).flatten(2).transpose(1, 2)
        return tok, (f, h, w)

    def unpatchify(self, x: torch.Tensor, grid) -> torch.Tensor:
        f, h, w = grid
        pt, ph, pw = self.patch_size
        B = x.shape[0]
        return x.view(B, f, h, w, pt, ph, pw, -1).permute(0, 7, 1, 4, 2, 5, 3, 6).reshape(B, -1, f * pt, h * ph, w * pw)


class VaceBlock(WanDiTBlock):
    def __init__(self, has_image_input, dim, heads, ffn_dim, eps=1e-6, block_id=0):
        super().__init__(has_image_input, dim, heads, ffn_dim, eps)
        self.block_id = block_id
        if block_id == 0:
            self.before_proj = nn.Linear(dim, dim)
        self.after_proj = nn.Linear(dim, dim)


class VaceWanModel(nn.Module):
    """Control branch: the control latents pass through their own copies of selected blocks; after each, a linear
    read-out is kept as the hint that the main model adds after the block of the same index."""

    def __init__(self, vace_layers=(0, 2, 4, 6, 8, 10, 12, 14, 16, 18, 20, 22, 24, 26, 28), vace_in_dim=96, patch_size=(1, 2, 2),
                 has_image_input=False, dim=1536, num_heads=12, ffn_dim=8960, eps=1e-6):
        super().__init__()
        self.vace_layers = tuple(vace_layers)
        self.vace_layers_mapping = {i: n for n, i in enumerate(self.vace_layers)}
        self.vace_blocks = nn.ModuleList([VaceBlock(has_image_input, dim, num_heads, ffn_dim, eps, block_id=i) for i in self.vace_layers])
        self.vace_patch_embedding = nn.Conv3d(vace_in_dim, dim, kernel_size=tuple(patch_size), stride=tuple(patch_size))

    def forward(self, x, vace_context, mod_tok, cu, cos, sin, ctx, cu_ctx, img=None, cu_img=None) -> List[torch.Tensor]:
        """``x [B*n, D]`` main tokens, ``vace_context [B, C, F, H, W]`` -> one hint ``[B*n, D]`` per control layer."""
        B = vace_context.shape[0]
        n = x.shape[0] // B
        c = self.vace_patch_embedding(vace_context.to(self.vace_patch_embedding.weight.dtype)).flatten(2).transpose(1, 2)
        if c.shape[1] < n:
            c = torch.cat([c, c.new_zeros(B, n - c.shape[1], c.shape[2])], 1)
        c = c.reshape(B * n, -1)
        hints = []
        for blk in self.vace_blocks:
            if blk.block_id == 0:
                c = F.linear(c, blk.before_proj.weight, blk.before_proj.bias) + x
            c = WanDiTBlock.forward(blk, c, mod_tok, cu, cos, sin, ctx, cu_ctx, img, cu_img)
            hints.append(F.linear(c, blk.after_proj.weight, blk.after_proj.bias))
        return hints


# ------------------------------------------------------------------------------------ wrapper
class WanVideoModel(nn.Module):
    """Children: ``dit`` and, when configured, ``vae``, ``text_encoder``, ``image_encoder``, ``motion_controller``,
    ``vace``.  ``forward`` is the training step's loss (flow matching on one random timestep per sample)."""

    config_class = WanVideoConfig
    _no_split_modules = ["WanDiTBlock", "VaceBlock"]

    def __init__(self, cfg: WanVideoConfig):
        super().__init__()
        self.config = cfg
        self.dit = WanDit(cfg)
        self.vae = WanVAE(**cfg.vae) if cfg.vae is not None else None
        self.text_encoder = WanTextEncoder(**cfg.text_encoder) if cfg.text_encoder is not None else None
        self.image_encoder = WanImageEncoder(**cfg.image_encoder) if cfg.image_encoder is not None else None
        self.motion_controller = WanMotionController(cfg.dit_freq_dim, cfg.dit_hidden_size) if cfg.motion_controller else None
        self.vace = None
        if cfg.vace is not None:
            kw = dict(patch_size=cfg.dit_patch_size, has_image_input=cfg.dit_has_image_input, dim=cfg.dit_hidden_size,
                      num_heads=cfg.dit_num_heads, ffn_dim=cfg.dit_intermediate_size, eps=cfg.dit_eps)
            kw.update(cfg.vace)
            self.vace = VaceWanModel(**kw)
        self.scheduler = FlowMatchScheduler(cfg.num_train_timesteps, cfg.shift)
        for m in self.dit.modules():
            if isinstance(m, nn.Linear):
                nn.init.xavier_uniform_(m.weight)
                if m.bias is not None:
                    nn.init.zeros_(m.bias)
        self.freeze_except()

    # ---- set-up -------------------------------------------------------------------------------------------
    def freeze_except(self, trainable_modules: Optional[str] = None):
        """Children named in the comma-separated list train; all others are frozen and kept in eval mode."""
        names = trainable_modules if trainable_modules is not None else (self.config.trainable_modules or "")
        keep = {n.strip() for n in names.split(",") if n.strip()}
        for name, child in self.named_children():
            child.requires_grad_(name in keep)
            child.train(name in keep)
        self._trainable_children = keep

    def train(self, mode: bool = True):
        super().train(mode)
        for name, child in self.named_children():
            if name not in getattr(self, "_trainable_children", {"dit"}):
                child.eval()
        return self

    def gradient_checkpointing_enable(self, **_):
        self.dit.gradient_checkpointing = True

    # ---- conditioning -------------------------------------------------------------------------------------
    @torch.no_grad()
    def encode_prompt(self, input_ids, attention_mask):
        if self.text_encoder is None:
            raise ValueError("prompt tokens were given but the model has no text_encoder (configure it or feed `context`)")
        return self.text_encoder.encode_prompt(input_ids, attention_mask)

    @torch.no_grad()
    def encode_video(self, video):
        """``[B, 3, T, H, W]`` (or a list of ``[3, T, H, W]``) in ``[-1, 1]`` -> latents."""
        if self.vae is None:
            raise ValueError("pixels were given but the model has no vae (configure it or feed `latents`)")
        return self.vae.encode(video)

    @torch.no_grad()
    def first_frame_condition(self, first_frame, num_frames: int, end_frame=None):
        """Image-to-video conditioning ``y``: a 4-row mask (which pixel frames are given) over the latents of a video
        that holds the given frame(s) and zeros elsewhere.  ``first_frame [B, 3, H, W]`` in ``[-1, 1]``."""
        B, _, H, W = first_frame.shape
        video = first_frame.new_zeros(B, 3, num_frames, H, W)
        video[:, :, 0] = first_frame
        s = self.vae.upsampling_factor
        msk = first_frame.new_zeros(B, num_frames, H // s, W // s)
        msk[:, 0] = 1
        if end_frame is not None:
            video[:, :, -1] = end_frame
            msk[:, -1] = 1
        msk = torch.cat([msk[:, :1].repeat_interleave(4, 1), msk[:, 1:]], 1)
        msk = msk.view(B, msk.shape[1] // 4, 4, H // s, W // s).transpose(1, 2)
        return torch.cat([msk, self.vae.encode(video).to(msk.dtype)], 1)

    # ---- denoiser -----------------------------------------------------------------------------------------
    def denoise(self, latents, timestep, context, y=None, clip_feature=None, reference_latents=None, vace_context=None, vace_scale=1.0,
                motion_bucket_id=None, control_camera_latents_input=None, token_timestep=None):
        """``latents [B, C, F, H, W]``, ``timestep [B]``, ``context [B, L, text_dim]`` -> prediction like ``latents``.
        ``token_timestep [B, f*h*w]`` gives every token its own timestep (clean first-frame tokens at 0)."""
        dit, cfg = self.dit, self.config
        dt = dit.patch_embedding.weight.dtype
        B = latents.shape[0]
        x = latents.to(dt)
        if y is not None and cfg.require_vae_embedding:
            x = torch.cat([x, y.to(dt)], 1)
        tok, (f, h, w) = dit.patchify(x, control_camera_latents_input)
        n_ref = 0
        if reference_latents is not None and cfg.dit_has_ref_conv:
            ref = reference_latents[:, :, 0] if reference_latents.dim() == 5 else reference_latents
            ref = dit.ref_conv(ref.to(dt)).flatten(2).transpose(1, 2)
            tok = torch.cat([ref, tok], 1)
            n_ref = ref.shape[1]
            f += 1
        n = tok.shape[1]
        xt = tok.reshape(B * n, -1)
        # timestep modulation, per sample or per token
        if token_timestep is not None:
            tt = token_timestep.reshape(-1)
            t_tok = dit.time_embedding(sinusoid_1d(dit.freq_dim, tt.float()).to(dt))
        else:
            t_tok = dit.time_embedding(sinusoid_1d(dit.freq_dim, timestep.float()).to(dt)).repeat_interleave(n, 0)
        mod_tok = dit.time_projection(t_tok).view(B * n, 6, -1)
        if motion_bucket_id is not None and self.motion_controller is not None:
            mb = self.motion_controller(motion_bucket_id.to(latents.device).reshape(-1)).view(-1, 6, dit.hidden_size)
            mod_tok = mod_tok + (mb.expand(B, -1, -1) if mb.shape[0] == 1 else mb).repeat_interleave(n, 0)
        L = context.shape[1]
        ctx = dit.text_embedding(context.reshape(B * L, -1).to(dt))
        cu = (torch.arange(B + 1, device=xt.device) * n).to(torch.int32)
        cu_ctx = (torch.arange(B + 1, device=xt.device) * L).to(torch.int32)
        img = cu_img = None
        if clip_feature is not None and cfg.require_clip_embedding and dit.has_image_input:
            e = dit.img_emb(clip_feature.to(dt))
            img, cu_img = e.reshape(-1, e.shape[-1]), (torch.arange(B + 1, device=xt.device) * e.shape[1]).to(torch.int32)
        cos, sin = rope_table_3d(dit.head_dim, f, h, w, xt.device)
        cos, sin = cos.repeat(B, 1), sin.repeat(B, 1)
        hints = None
        if vace_context is not None and self.vace is not None:
            hints = self.vace(xt, vace_context, mod_tok, cu, cos, sin, ctx, cu_ctx, img, cu_img)
        for i, blk in enumerate(dit.blocks):
            if dit.gradient_checkpointing and self.training:
                xt = torch.utils.checkpoint.checkpoint(blk, xt, mod_tok, cu, cos, sin, ctx, cu_ctx, img, cu_img, use_reentrant=False)
            else:
                xt = blk(xt, mod_tok, cu, cos, sin, ctx, cu_ctx, img, cu_img)
            if hints is not None and i in self.vace.vace_layers_mapping:
                xt = xt + hints[self.vace.vace_layers_mapping[i]] * vace_scale
        out = dit.head(xt, t_tok).view(B, n, -1).float()
        if n_ref:
            out, f = out[:, n_ref:], f - 1
        return dit.unpatchify(out, (f, h, w))

    # ---- training step ------------------------------------------------------------------------------------
    def forward(self, latents=None, context=None, video=None, input_ids=None, attention_mask=None, input_image=None, clip_feature=None,
                y=None, timestep_index=None, noise=None, **cond) -> Dict[str, Any]:
        """Flow matching: noise the latents to a random timestep, predict ``noise - latents``, weighted MSE.

        Accepts stored ``latents`` / ``context`` or raw ``video`` (``[B, 3, T, H, W]`` in ``[-1, 1]``) / ``input_ids``.
        With ``fuse_vae_embedding_in_latents`` and an ``input_image`` the first latent frame is given clean, its tokens
        run at timestep 0 (``seperated_timestep``) and it is left out of the loss."""
        cfg = self.config
        if video is not None and video.dim() == 5 and video.shape[-1] == 3 and video.shape[1] != 3:
            video = video.permute(0, 4, 1, 2, 3)  # the data plane's [B, T, H, W, C]
        if video is not None and input_image is None and self.vae is not None and (
                cfg.fuse_vae_embedding_in_latents or cfg.require_vae_embedding or cfg.require_clip_embedding):
            input_image = video[:, :, 0]  # the clip's first frame conditions the sample, as in the reference's trainer
        if latents is None:
            latents = self.encode_video(video)
        if context is None:
            context = self.encode_prompt(input_ids, attention_mask)
        latents = latents.float()
        B = latents.shape[0]
        dev = latents.device
        idx = timestep_index if timestep_index is not None else torch.randint(0, self.scheduler.n, (B,), device=dev)
        noise = torch.randn_like(latents) if noise is None else noise.float()
        noisy = self.scheduler.add_noise(latents, noise, idx.cpu())
        target = self.scheduler.training_target(latents, noise)
        t = self.scheduler.timesteps.to(dev)[idx]
        token_t, loss_mask = None, None
        if input_image is not None and self.vae is not None:
            if cfg.require_vae_embedding and y is None:
                y = self.first_frame_condition(input_image, 1 + 4 * (latents.shape[2] - 1))
            if cfg.require_clip_embedding and clip_feature is None and self.image_encoder is not None:
                clip_feature = self.image_encoder.encode_image([input_image])
            if cfg.fuse_vae_embedding_in_latents:
                noisy = noisy.clone()
                noisy[:, :, :1] = self.vae.encode(input_image[:, :, None]).float()
                loss_mask = torch.ones_like(latents[:, :1])
                loss_mask[:, :, :1] = 0
                if cfg.seperated_timestep:
                    pt, ph, pw = self.dit.patch_size
                    f, h, w = latents.shape[2] // pt, latents.shape[3] // ph, latents.shape[4] // pw
                    token_t = t.view(B, 1, 1, 1).expand(B, f, h, w).clone()
                    token_t[:, 0] = 0
                    token_t = token_t.reshape(B, -1)
        pred = self.denoise(noisy, t, context, y=y, clip_feature=clip_feature, token_timestep=token_t, **cond)
        wgt = self.scheduler.training_weight(idx.cpu(), dev).view(B, 1, 1, 1, 1)
        err = wgt * (pred - target) ** 2
        loss = err.mean() if loss_mask is None else (err * loss_mask).sum() / (loss_mask.expand_as(err).sum().clamp(min=1))
        return {"loss": loss, "noise_pred": pred}

    def convert_hf_state_dict(self, sd: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        """Released DiT checkpoints hold the transformer's keys without a prefix; the wrapper's own layout prefixes every
        child (``dit.``, ``vae.``, ...).  Keys that already carry a child prefix pass through."""
        children = {"dit", "vae", "text_encoder", "image_encoder", "motion_controller", "vace"}
        return {(k if k.split(".", 1)[0] in children else "dit." + k): v for k, v in sd.items()}
