"""Minimal vision-language model: a SigLIP-style patch encoder, an MLP projector and a packed decoder
(reference: src/lmms_engine/models/nanovlm/modeling_nanovlm.py:25-173, configuration_nanovlm.py:6-69).

The reference assembles it from two ``transformers`` models; here the encoder runs on the engine's own
kernels (GEMM, LayerNorm, non-causal varlen attention over the patches of each image) and the decoder
is ``DecoderLM`` on the flat token stream.  Images arrive NaFlex-style as already flattened patches
``pixel_values [n_patches_total, C*p*p]`` with ``spatial_shapes [n_images, 2]`` (patch rows, columns);
every image contributes ``rows*cols`` feature rows that replace its ``image_token_id`` placeholders in
order.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field, fields
from typing import Any, Dict, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import attention as attn_ops
from ..ops import gemm as gemm_ops
from .decoder_lm import DecoderConfig, DecoderLM
from .vision import LayerNorm


@dataclass
class NanoVisionConfig:
    hidden_size: int = 768
    intermediate_size: int = 3072
    num_hidden_layers: int = 12
    num_attention_heads: int = 12
    num_channels: int = 3
    patch_size: int = 16
    num_patches: int = 256  # side*side of the learned position grid, interpolated to each image's shape
    layer_norm_eps: float = 1e-6
    hidden_act: str = "gelu_pytorch_tanh"

    @classmethod
    def from_dict(cls, d):
        known = {f.name for f in fields(cls)}
        return cls(**{k: v for k, v in (d or {}).items() if k in known})


@dataclass
class NanovlmConfig:
    model_type: str = "nanovlm"
    text_config: Any = None
    vision_config: Any = None
    image_token_id: Optional[int] = None
    projector_hidden_size: Optional[int] = None
    projector_num_layers: int = 2
    projector_hidden_act: str = "gelu"
    vision_feature_dim: Optional[int] = None
    image_token_count: int = 256
    extra: Dict[str, Any] = field(default_factory=dict)

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "NanovlmConfig":
        d = dict(d)
        text = d.pop("text_config", None) or {}
        vis = d.pop("vision_config", None) or {}
        known = {f.name for f in fields(cls)}
        kw = {k: v for k, v in d.items() if k in known}
        kw["extra"] = {k: v for k, v in d.items() if k not in known}
        cfg = cls(**kw)
        cfg.text_config = text if isinstance(text, DecoderConfig) else DecoderConfig.from_dict({"model_type": "qwen3", **text})
        cfg.vision_config = vis if isinstance(vis, NanoVisionConfig) else NanoVisionConfig.from_dict(vis)
        cfg.vision_feature_dim = int(cfg.vision_feature_dim or cfg.vision_config.hidden_size)
        return cfg

    def to_dict(self):
        return {"model_type": self.model_type, "text_config": self.text_config.to_dict(),
                "vision_config": {f.name: getattr(self.vision_config, f.name) for f in fields(self.vision_config)},
                "image_token_id": self.image_token_id, "projector_hidden_size": self.projector_hidden_size,
                "projector_num_layers": self.projector_num_layers, "projector_hidden_act": self.projector_hidden_act,
                "vision_feature_dim": self.vision_feature_dim, "image_token_count": self.image_token_count, **self.extra}

    @property
    def vocab_size(self):
        return self.text_config.vocab_size


def _act(name: str, x):
    if "tanh" in name or name in ("gelu_new", "gelu_fast"):
        return F.gelu(x, approximate="tanh")
    if name in ("silu", "swish"):
        return F.silu(x)
    if name == "relu":
        return F.relu(x)
    return F.gelu(x)


class _EncoderLayer(nn.Module):
    def __init__(self, c: NanoVisionConfig):
        super().__init__()
        d = c.hidden_size
        self.heads, self.head_dim, self.act = c.num_attention_heads, d // c.num_attention_heads, c.hidden_act
        self.layer_norm1, self.layer_norm2 = LayerNorm(d, c.layer_norm_eps), LayerNorm(d, c.layer_norm_eps)
        self.qkv = nn.Linear(d, 3 * d)
        self.out_proj = nn.Linear(d, d)
        self.fc1, self.fc2 = nn.Linear(d, c.intermediate_size), nn.Linear(c.intermediate_size, d)

    def forward(self, x, cu):
        P = x.shape[0]
        qkv = gemm_ops.linear(self.layer_norm1(x), self.qkv.weight, self.qkv.bias).view(P, 3, self.heads, self.head_dim)
        o = attn_ops.varlen_attn(qkv[:, 0], qkv[:, 1], qkv[:, 2], cu, cu, causal=False, softmax_scale=1.0 / math.sqrt(self.head_dim))
        x = x + gemm_ops.linear(o.reshape(P, -1), self.out_proj.weight, self.out_proj.bias)
        h = _act(self.act, gemm_ops.linear(self.layer_norm2(x), self.fc1.weight, self.fc1.bias))
        return x + gemm_ops.linear(h, self.fc2.weight, self.fc2.bias)


class NanoVisionEncoder(nn.Module):
    def __init__(self, c: NanoVisionConfig):
        super().__init__()
        self.cfg = c
        self.patch_embedding = nn.Linear(c.num_channels * c.patch_size ** 2, c.hidden_size)
        self.side = int(round(math.sqrt(c.num_patches)))
        self.position_embedding = nn.Embedding(self.side * self.side, c.hidden_size)
        self.layers = nn.ModuleList([_EncoderLayer(c) for _ in range(c.num_hidden_layers)])
        self.post_layernorm = LayerNorm(c.hidden_size, c.layer_norm_eps)

    def positions(self, shapes):
        """Learned grid resized (bilinear, as NaFlex does) to every image's patch grid."""
        grid = self.position_embedding.weight.view(1, self.side, self.side, -1).permute(0, 3, 1, 2).float()
        out = []
        for h, w in shapes:
            if (h, w) == (self.side, self.side):
                out.append(self.position_embedding.weight)
            else:
                p = F.interpolate(grid, size=(h, w), mode="bilinear", align_corners=False, antialias=True)
                out.append(p[0].permute(1, 2, 0).reshape(h * w, -1).to(self.position_embedding.weight.dtype))
        return torch.cat(out, 0)

    def forward(self, pixel_values: torch.Tensor, spatial_shapes) -> torch.Tensor:
        shapes = [(int(h), int(w)) for h, w in (spatial_shapes.tolist() if torch.is_tensor(spatial_shapes) else spatial_shapes)]
        w = self.patch_embedding.weight
        x = gemm_ops.linear(pixel_values.to(w.dtype), w, self.patch_embedding.bias) + self.positions(shapes).to(w.dtype)
        lens = torch.tensor([0] + [h * w_ for h, w_ in shapes], device=x.device)
        cu = torch.cumsum(lens, 0).to(torch.int32)
        for layer in self.layers:
            x = layer(x, cu)
        return self.post_layernorm(x)


class Nanovlm(nn.Module):
    config_class = NanovlmConfig
    _no_split_modules = ["DecoderLayer", "_EncoderLayer"]

    def __init__(self, cfg: NanovlmConfig):
        super().__init__()
        self.config = cfg
        self.language_model = DecoderLM(cfg.text_config)
        self.vision_model = NanoVisionEncoder(cfg.vision_config)
        hid, out = cfg.projector_hidden_size or cfg.text_config.hidden_size, cfg.text_config.hidden_size
        if cfg.projector_num_layers <= 1:
            self.multi_modal_projector = nn.Linear(cfg.vision_feature_dim, out)
        else:
            self.multi_modal_projector = nn.Sequential(nn.Linear(cfg.vision_feature_dim, hid), nn.GELU(), nn.Linear(hid, out))
        self.projector_act = cfg.projector_hidden_act

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

    def project(self, feats):
        p = self.multi_modal_projector
        if isinstance(p, nn.Linear):
            return gemm_ops.linear(feats, p.weight, p.bias)
        h = _act(self.projector_act, gemm_ops.linear(feats, p[0].weight, p[0].bias))
        return gemm_ops.linear(h, p[2].weight, p[2].bias)

    def forward(self, input_ids=None, labels=None, attention_mask=None, pixel_values=None, spatial_shapes=None,
                cu_seqlens=None, position_ids=None, **kw):
        from .decoder_lm import unpad_batch

        ids, lab, cu, pos = input_ids, labels, cu_seqlens, position_ids
        if ids.dim() == 2:  # padded [n, L] batch -> flat stream
            ids, lab, pos, cu, _ = unpad_batch(ids, attention_mask if attention_mask is not None else torch.ones_like(ids), lab)
        else:
            ids, lab, pos, cu, _ = self.language_model.prepare_packed(ids, None, lab, pos, cu)
        emb = self.get_input_embeddings()(ids)
        if pixel_values is not None and pixel_values.numel() > 0:
            feats = self.project(self.vision_model(pixel_values, spatial_shapes)).to(emb.dtype)
            mask = ids == self.config.image_token_id
            # the k-th placeholder takes the k-th feature row (counts must match; checked without a host sync
            # by clamping, a mismatch shows up as a loss that the data checks catch)
            src = (torch.cumsum(mask, 0) - 1).clamp(min=0, max=max(feats.shape[0] - 1, 0))
            emb = torch.where(mask.unsqueeze(-1), feats.index_select(0, src), emb)
        return self.language_model(inputs_embeds=emb, labels=lab, cu_seqlens=cu, position_ids=pos)
