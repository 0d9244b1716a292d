"""LLaVA-OneVision: SigLIP tower on fixed-size tiles, two-layer projector, any-resolution packing of the
tile features with a learned newline vector, Qwen2 decoder on the packed stream
(``model_type: llava_onevision``; the reference patches the ``transformers`` classes,
src/lmms_engine/models/llava_onevision/monkey_patch.py, llava_onevision_ops.py).

Behaviour reproduced from the upstream model: an image arrives as ``1 + rows*cols`` tiles (a resized base
view and the tiles of the best-fitting grid resolution); tile features are laid out on the grid, cropped
back to the image's aspect ratio, shrunk bilinearly when they exceed ``anyres_max_N`` tile areas, a newline
vector ends every row, and the base view's features come first.  Video frames are pooled 2x bilinearly and
a single newline ends the clip.  Features replace the image / video placeholders of the stream in order.
Parameter names follow the hub checkpoints.
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
from .decoder_lm import DecoderConfig, DecoderLM, unpad_batch
from .vision import LayerNorm


# ------------------------------------------------------------------------------- any-resolution geometry
def select_best_resolution(original_size: Tuple[int, int], resolutions: List[Tuple[int, int]]) -> Tuple[int, int]:
    """(height, width) among ``resolutions`` that keeps most of the image and wastes least area."""
    oh, ow = original_size
    best, best_eff, best_waste = None, 0, float("inf")
    for h, w in resolutions:
        scale = min(w / ow, h / oh)
        eff = min(int(ow * scale) * int(oh * scale), ow * oh)
        waste = w * h - eff
        if eff > best_eff or (eff == best_eff and waste < best_waste):
            best, best_eff, best_waste = (h, w), eff, waste
    return best


def anyres_grid(image_size, pinpoints, tile: int) -> Tuple[int, int]:
    h, w = select_best_resolution(tuple(int(x) for x in image_size), [tuple(p) for p in pinpoints])
    return h // tile, w // tile


def unpad_features(t: torch.Tensor, original_size) -> torch.Tensor:
    """``t [C, H, W]`` laid out over the padded canvas -> the part that covers the original image."""
    oh, ow = (int(x) for x in original_size)
    ch, cw = t.shape[1:]
    if ow / oh > cw / ch:
        new_h = int(round(oh * (cw / ow), 7))
        pad = (ch - new_h) // 2
        return t[:, pad:ch - pad, :]
    new_w = int(round(ow * (ch / oh), 7))
    pad = (cw - new_w) // 2
    return t[:, :, pad:cw - pad]


def packed_image_tokens(image_size, pinpoints, tile: int, side: int, max_tiles: int = 9) -> int:
    """Number of feature rows an image of ``image_size`` (h, w) becomes (what the processor must reserve)."""
    gh, gw = anyres_grid(image_size, pinpoints, tile)
    t = torch.empty((1, gh * side, gw * side), device="meta")
    _, ch, cw = unpad_features(t, image_size).shape
    ratio = math.sqrt(ch * cw / (max_tiles * side * side))
    if ratio > 1.1:
        ch, cw = int(ch // ratio), int(cw // ratio)
    return side * side + ch * (cw + 1)


# ------------------------------------------------------------------------------- config
@dataclass
class SiglipConfig:
    hidden_size: int = 1152
    intermediate_size: int = 4304
    num_hidden_layers: int = 26
    num_attention_heads: int = 16
    num_channels: int = 3
    image_size: int = 384
    patch_size: int = 14
    layer_norm_eps: float = 1e-6
    hidden_act: str = "gelu_pytorch_tanh"

    @classmethod
    def from_dict(cls, d):
        known = {f.name for f in fields(cls)}
        return cls(**{k: v for k, v in (d or {}).items() if k in known})


@dataclass
class LlavaOnevisionConfig:
    model_type: str = "llava_onevision"
    text_config: Any = None
    vision_config: Any = None
    image_token_index: int = 151646
    video_token_index: int = 151647
    projector_hidden_act: str = "gelu"
    vision_feature_select_strategy: str = "full"
    vision_feature_layer: int = -1
    vision_aspect_ratio: str = "anyres_max_9"
    image_grid_pinpoints: Optional[List[List[int]]] = None
    multimodal_projector_bias: bool = True
    tie_word_embeddings: bool = False
    extra: Dict[str, Any] = field(default_factory=dict)

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "LlavaOnevisionConfig":
        d = dict(d)
        text, vis = dict(d.pop("text_config", None) or {}), dict(d.pop("vision_config", None) or {})
        known = {f.name for f in fields(cls)}
        kw = {k: v for k, v in d.items() if k in known}
        kw["extra"] = {k: v for k, v in d.items() if k not in known}
        cfg = cls(**kw)
        text.setdefault("model_type", "qwen2")
        text["tie_word_embeddings"] = bool(d.get("tie_word_embeddings", False))
        cfg.text_config = DecoderConfig.from_dict(text)
        cfg.vision_config = SiglipConfig.from_dict(vis)
        if cfg.image_grid_pinpoints is None:
            s = cfg.vision_config.image_size
            cfg.image_grid_pinpoints = [[s * i, s * j] for i in range(1, 7) for j in range(1, 7)]
        if cfg.vision_feature_layer != -1 or cfg.vision_feature_select_strategy != "full":
            raise ValueError("only the last SigLIP layer with the 'full' selection is supported")
        return cfg

    def to_dict(self):
        d = {f.name: getattr(self, f.name) for f in fields(self) if f.name not in ("text_config", "vision_config", "extra")}
        d["text_config"] = self.text_config.to_dict()
        d["vision_config"] = {"model_type": "siglip_vision_model", **{f.name: getattr(self.vision_config, f.name) for f in fields(self.vision_config)}}
        d["architectures"] = ["LlavaOnevisionForConditionalGeneration"]
        d.update(self.extra)
        return d

    @property
    def vocab_size(self):
        return self.text_config.vocab_size

    def __getattr__(self, name):
        if name in ("text_config", "vision_config") or name.startswith("__"):
            raise AttributeError(name)
        return getattr(self.text_config, name)


# ------------------------------------------------------------------------------- SigLIP tower
class _SiglipAttention(nn.Module):
    def __init__(self, d, heads):
        super().__init__()
        self.heads, self.head_dim = heads, d // heads
        self.q_proj, self.k_proj, self.v_proj, self.out_proj = (nn.Linear(d, d) for _ in range(4))

    def forward(self, x, cu):
        P = x.shape[0]
        w = torch.cat([self.q_proj.weight, self.k_proj.weight, self.v_proj.weight], 0)
        b = torch.cat([self.q_proj.bias, self.k_proj.bias, self.v_proj.bias], 0)
        qkv = gemm_ops.linear(x, w, b).view(P, 3, self.heads, self.head_dim)
        o = attn_ops.varlen_attn(qkv[:, 0], qkv[:, 1], qkv[:, 2], cu, cu, causal=False, softmax_scale=self.head_dim ** -0.5)
        return gemm_ops.linear(o.reshape(P, -1), self.out_proj.weight, self.out_proj.bias)


class _SiglipMLP(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.fc1, self.fc2, self.act = nn.Linear(c.hidden_size, c.intermediate_size), nn.Linear(c.intermediate_size, c.hidden_size), c.hidden_act

    def forward(self, x):
        h = gemm_ops.linear(x, self.fc1.weight, self.fc1.bias)
        h = F.gelu(h, approximate="tanh") if "tanh" in self.act else F.gelu(h)
        return gemm_ops.linear(h, self.fc2.weight, self.fc2.bias)


class SiglipEncoderLayer(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.layer_norm1, self.layer_norm2 = LayerNorm(c.hidden_size, c.layer_norm_eps), LayerNorm(c.hidden_size, c.layer_norm_eps)
        self.self_attn, self.mlp = _SiglipAttention(c.hidden_size, c.num_attention_heads), _SiglipMLP(c)

    def forward(self, x, cu):
        x = x + self.self_attn(self.layer_norm1(x), cu)
        return x + self.mlp(self.layer_norm2(x))


class _Embeddings(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.patch_embedding = nn.Conv2d(c.num_channels, c.hidden_size, kernel_size=c.patch_size, stride=c.patch_size, padding="valid")
        self.side = c.image_size // c.patch_size
        self.position_embedding = nn.Embedding(self.side ** 2, c.hidden_size)
        self.patch = c.patch_size

    def forward(self, pixel_values):  # [n, C, S, S] -> [n * side^2, hidden]: the strided convolution as one GEMM
        n, C, S, _ = pixel_values.shape
        p, side = self.patch, self.side
        x = pixel_values[:, :, : side * p, : side * p].reshape(n, C, side, p, side, p).permute(0, 2, 4, 1, 3, 5).reshape(n * side * side, C * p * p)
        w = self.patch_embedding.weight.view(self.patch_embedding.weight.shape[0], -1)
        x = gemm_ops.linear(x.to(w.dtype), w, self.patch_embedding.bias)
        return x + self.position_embedding.weight.repeat(n, 1).to(x.dtype)


class _Encoder(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.layers = nn.ModuleList([SiglipEncoderLayer(c) for _ in range(c.num_hidden_layers)])


class _VisionModel(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.embeddings, self.encoder = _Embeddings(c), _Encoder(c)
        self.post_layernorm = LayerNorm(c.hidden_size, c.layer_norm_eps)  # in the checkpoints; the last layer's output is used before it


class SiglipTower(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.vision_model = _VisionModel(c)

    def forward(self, pixel_values):
        """``[n, C, S, S]`` -> last encoder layer output ``[n, side^2, hidden]`` (tiles attend only within themselves)."""
        vm = self.vision_model
        n = pixel_values.shape[0]
        x = vm.embeddings(pixel_values)
        per = vm.embeddings.side ** 2
        cu = (torch.arange(n + 1, device=x.device) * per).to(torch.int32)
        for layer in vm.encoder.layers:
            x = layer(x, cu)
        return x.view(n, per, -1)


class _MMProjector(nn.Module):
    def __init__(self, d_in, d_out, bias=True):
        super().__init__()
        self.linear_1, self.linear_2 = nn.Linear(d_in, d_out, bias=bias), nn.Linear(d_out, d_out, bias=bias)

    def forward(self, x):
        h = F.gelu(gemm_ops.linear(x, self.linear_1.weight, self.linear_1.bias))
        return gemm_ops.linear(h, self.linear_2.weight, self.linear_2.bias)


# ------------------------------------------------------------------------------- model
class LlavaOnevision(nn.Module):
    config_class = LlavaOnevisionConfig
    _no_split_modules = ["DecoderLayer", "SiglipEncoderLayer"]

    def __init__(self, cfg: LlavaOnevisionConfig):
        super().__init__()
        self.config = cfg
        self.vision_tower = SiglipTower(cfg.vision_config)
        self.multi_modal_projector = _MMProjector(cfg.vision_config.hidden_size, cfg.text_config.hidden_size, cfg.multimodal_projector_bias)
        self.image_newline = nn.Parameter(torch.randn(cfg.text_config.hidden_size) / math.sqrt(cfg.text_config.hidden_size))
        self.language_model = DecoderLM(cfg.text_config)

    @property
    def sp_group(self):
        return self.language_model.sp_group

    @sp_group.setter
    def sp_group(self, g):
        self.language_model.sp_group = g

    def gradient_checkpointing_enable(self, *a, **k):
        self.language_model.gradient_checkpointing_enable()

    def get_input_embeddings(self):
        return self.language_model.model.embed_tokens

    # ---- features --------------------------------------------------------------------------------
    def image_features(self, pixel_values, image_sizes, batch_num_images=None) -> torch.Tensor:
        cfg = self.config
        tile, side = cfg.vision_config.image_size, cfg.vision_config.image_size // cfg.vision_config.patch_size
        sizes = image_sizes.tolist() if torch.is_tensor(image_sizes) else [list(s) for s in image_sizes]
        if batch_num_images is None:
            patching = [True] * len(sizes)
        else:
            nums = batch_num_images.tolist() if torch.is_tensor(batch_num_images) else list(batch_num_images)
            patching = [n == 1 for n in nums for _ in range(n)]
        grids = [anyres_grid(s, cfg.image_grid_pinpoints, tile) if p else None for s, p in zip(sizes, patching)]
        counts = [1 + g[0] * g[1] if g is not None else 1 for g in grids]
        if pixel_values.dim() == 5:
            pixel_values = torch.cat([pv[:c] for pv, c in zip(pixel_values, counts)], 0)
        feats = self.multi_modal_projector(self.vision_tower(pixel_values).flatten(0, 1)).view(pixel_values.shape[0], side * side, -1)
        max_tiles = int(cfg.vision_aspect_ratio.replace("anyres_max_", ""))
        out, start = [], 0
        nl = self.image_newline.to(feats.dtype)
        for size, grid, c in zip(sizes, grids, counts):
            f = feats[start:start + c]
            start += c
            if c > 1:
                base, rest = f[0], f[1:]
                gh, gw = grid
                canvas = rest.view(gh, gw, side, side, -1).permute(4, 0, 2, 1, 3).reshape(-1, gh * side, gw * side)
                canvas = unpad_features(canvas, size)
                _, ch, cw = canvas.shape
                ratio = math.sqrt(ch * cw / (max_tiles * side * side))
                if ratio > 1.1:
                    canvas = F.interpolate(canvas[None], [int(ch // ratio), int(cw // ratio)], mode="bilinear")[0]
                canvas = torch.cat([canvas, nl[:, None, None].expand(-1, canvas.shape[1], 1)], -1)
                out.append(torch.cat([base, canvas.flatten(1, 2).transpose(0, 1)], 0))
            else:
                out.append(torch.cat([f[0], nl[None]], 0))
        return torch.cat(out, 0)

    def video_features(self, pixel_values_videos) -> torch.Tensor:
        b, t = pixel_values_videos.shape[:2]
        side = self.config.vision_config.image_size // self.config.vision_config.patch_size
        f = self.multi_modal_projector(self.vision_tower(pixel_values_videos.flatten(0, 1)).flatten(0, 1)).view(b * t, side, side, -1)
        f = F.interpolate(f.permute(0, 3, 1, 2), size=[math.ceil(side / 2)] * 2, mode="bilinear").permute(0, 2, 3, 1)
        f = f.reshape(b, -1, f.shape[-1])
        nl = self.image_newline.to(f.dtype)[None, None].expand(b, 1, -1)
        return torch.cat([f, nl], 1).flatten(0, 1)

    def forward(self, input_ids=None, labels=None, attention_mask=None, pixel_values=None, image_sizes=None,
                pixel_values_videos=None, batch_num_images=None, cu_seqlens=None, position_ids=None, **kw):
        ids, lab, cu, pos = input_ids, labels, cu_seqlens, position_ids
        if ids.dim() == 2:
            ids, lab, pos, cu, _ = unpad_batch(ids, attention_mask if attention_mask is not None else torch.ones_like(ids), lab)
        else:
            ids, lab, pos, cu, _ = self.language_model.prepare_packed(ids, None, lab, pos, cu)
        emb = self.get_input_embeddings()(ids)
        for feats, tok in ((self.image_features(pixel_values, image_sizes, batch_num_images) if pixel_values is not None and pixel_values.numel() else None,
                            self.config.image_token_index),
                           (self.video_features(pixel_values_videos) if pixel_values_videos is not None and pixel_values_videos.numel() else None,
                            self.config.video_token_index)):
            if feats is None:
                continue
            m = ids == tok
            src = (torch.cumsum(m, 0) - 1).clamp(min=0, max=max(feats.shape[0] - 1, 0))
            emb = torch.where(m.unsqueeze(-1), feats.to(emb.dtype).index_select(0, src), emb)
        return self.language_model(inputs_embeds=emb, labels=lab, cu_seqlens=cu, position_ids=pos)

    # ---- hub names ----------------------------------------------------------------------------------
    def convert_hf_state_dict(self, sd):
        out = {}
        for k, v in sd.items():
            if k.startswith("model.language_model."):
                out["language_model.model." + k[len("model.language_model."):]] = v
            elif k.startswith("lm_head."):
                out["language_model." + k] = v
            elif k.startswith("model."):
                k2 = k[len("model."):]
                if ".vision_model.head." in k2:
                    continue  # pooling head of the tower: not used by the language model path
                out[k2] = v
            elif k.startswith("language_model.model.") or k.startswith("language_model.lm_head."):
                out[k] = v
            else:
                out[k] = v
        return out
