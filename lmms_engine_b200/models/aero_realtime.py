"""aero_realtime: a streaming audio + vision language model over a vision-language backbone family
(``qwen3_vl``, ``qwen3_vl_moe``, ``qwen3_5``, ``qwen3_5_moe``).

* the causal streaming audio encoder (``models/audio.py``: causal convolutions, rotary sliding-window attention)
  runs on every clip; ``downsample_factor`` consecutive encoder frames are concatenated into one row and mapped to
  the decoder width by a two-layer projector without biases;
* the token stream has a parallel **text stream** (``text_stream_ids``): at audio positions it carries the realtime
  tokens (pad / speak / boundaries / transcript) whose embeddings the audio rows are ADDED to; elsewhere it mirrors
  ``input_ids``.  Placeholders for images, videos and audio are located in ``input_ids``;
* image / video features overwrite their placeholders as in the backbone family; positions are the family's
  multimodal rotary positions (audio positions advance like text).

Reference: src/lmms_engine/models/aero_realtime/modeling_aero_realtime.py:110-148 (projector), :380-440 (audio features),
:460-676 (forward), configuration_aero_realtime.py:187-300, backbone_registry.py.  The reference encoder's variants (LayerNorm, GELU MLP, symmetric
convolution padding, attention without causality) are configuration fields of the audio encoder (``models/audio.py``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import gemm as gemm_ops
from .audio import VoxtralRealtimeEncoder, VoxtralRealtimeEncoderConfig
from .vl import VLConfig, VLModel

FAMILIES = ("qwen3_vl", "qwen3_vl_moe", "qwen3_5", "qwen3_5_moe")


@dataclass
class AeroRealtimeConfig(VLConfig):
    backbone_family: str = "qwen3_vl"
    audio_config: Any = None
    projector_hidden_act: str = "gelu"
    downsample_factor: int = 4
    audio_length_per_tok: int = 8
    audio_token_id: int = 151671

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "AeroRealtimeConfig":
        d = dict(d)
        family = d.pop("backbone_family", "qwen3_vl")
        if family not in FAMILIES:
            raise ValueError(f"unknown backbone_family={family}; expected one of {FAMILIES}")
        audio = dict(d.pop("audio_config", None) or {})
        own = {k: d.pop(k) for k in ("projector_hidden_act", "downsample_factor", "audio_length_per_tok") if k in d}
        for a, b in (("image_token_index", "image_token_id"), ("video_token_index", "video_token_id"),
                     ("vision_start_token_index", "vision_start_token_id"), ("audio_token_index", "audio_token_id")):
            if a in d:
                d.setdefault(b, d.pop(a))
        audio_tok = d.pop("audio_token_id", None)
        d["model_type"] = family
        base = VLConfig.from_dict(d)
        cfg = cls(**{f: getattr(base, f) for f in VLConfig.__dataclass_fields__}, backbone_family=family, **own)
        cfg.model_type = "aero_realtime"
        cfg.audio_config = VoxtralRealtimeEncoderConfig.from_dict(audio)
        if audio_tok is not None:
            cfg.audio_token_id = int(audio_tok)
        return cfg

    @property
    def is_qwen3(self) -> bool:
        return True

    def to_dict(self) -> Dict[str, Any]:
        d = super().to_dict()
        d.update(model_type="aero_realtime", architectures=["AeroRealtimeForConditionalGeneration"],
                 backbone_family=self.backbone_family, audio_config=self.audio_config.to_dict(),
                 projector_hidden_act=self.projector_hidden_act, downsample_factor=self.downsample_factor,
                 audio_length_per_tok=self.audio_length_per_tok, audio_token_index=self.audio_token_id,
                 image_token_index=self.image_token_id, video_token_index=self.video_token_id)
        return d


class AeroRealtimeProjector(nn.Module):
    def __init__(self, cfg: AeroRealtimeConfig):
        super().__init__()
        H = cfg.text_config.hidden_size
        self.linear_1 = nn.Linear(cfg.audio_config.hidden_size * cfg.downsample_factor, H, bias=False)
        self.linear_2 = nn.Linear(H, H, bias=False)
        self.act = cfg.projector_hidden_act

    def forward(self, x):
        h = gemm_ops.linear(x, self.linear_1.weight, None)
        h = F.gelu(h) if "gelu" in self.act else F.silu(h)
        return gemm_ops.linear(h, self.linear_2.weight, None)


class AeroRealtimeModel(VLModel):
    config_class = AeroRealtimeConfig
    _no_split_modules = VLModel._no_split_modules + ["VoxtralEncoderLayer"]

    def __init__(self, cfg: AeroRealtimeConfig):
        base = VLConfig(**{f: getattr(cfg, f) for f in VLConfig.__dataclass_fields__})
        base.model_type = cfg.backbone_family
        super().__init__(base)
        self.config = cfg
        self.audio_tower = VoxtralRealtimeEncoder(cfg.audio_config)
        self.multi_modal_projector = AeroRealtimeProjector(cfg)
        self._rt = None

    def audio_rows(self, input_features, mask, stream_cache=None):
        """Projected audio rows of all clips, clip after clip: ``frames // downsample_factor`` rows per clip.  With
        ``stream_cache`` (``audio_tower.new_stream()``) the features are the NEXT piece of one running clip and the
        encoder continues from the cache instead of starting a clip."""
        df = self.config.downsample_factor
        if stream_cache is not None:
            hidden = self.audio_tower.stream(input_features.reshape(input_features.shape[-2], input_features.shape[-1]), stream_cache)
            keep = hidden.shape[0] // df * df
            return self.multi_modal_projector(hidden[:keep].reshape(keep // df, -1))
        T = input_features.shape[-1]
        if mask is not None and mask.shape[-1] != T:
            # frame-level mask (after the stride-2 convolution): f frames cover 2 f mel frames
            lens = mask.sum(-1).long() * 2
            mask = (torch.arange(T, device=mask.device)[None, :] < lens[:, None]).to(mask.dtype)
        out = self.audio_tower(input_features, mask)
        hidden, frames = out["last_hidden_state"], out["frame_lengths"].tolist()
        rows, at = [], 0
        for f in frames:
            keep = f // df * df
            rows.append(hidden[at:at + keep].reshape(keep // df, -1))
            at += f
        return self.multi_modal_projector(torch.cat(rows, 0))

    def embed_multimodal(self, ids, pixel_values, image_grid_thw, pixel_values_videos, video_grid_thw, embed_ids=None):
        stream, feats, mask, audio_cache = self._rt or (None, None, None, None)
        emb, deep, idx = super().embed_multimodal(ids, pixel_values, image_grid_thw, pixel_values_videos, video_grid_thw,
                                                  embed_ids=stream)
        if feats is not None:
            rows = self.audio_rows(feats.to(emb.dtype), mask, audio_cache)
            m = ids == self.config.audio_token_id
            # the k-th audio position receives the k-th row, added to the text-stream embedding
            src = (torch.cumsum(m, 0) - 1).clamp(min=0, max=max(rows.shape[0] - 1, 0))
            emb = emb + torch.where(m.unsqueeze(-1), rows.to(emb.dtype).index_select(0, src), torch.zeros_like(emb))
        return emb, deep, idx

    def forward(self, input_ids=None, attention_mask=None, text_stream_ids=None, input_features=None,
                audio_attention_mask=None, feature_attention_mask=None, audio_stream_cache=None, **kw):
        stream = None
        if text_stream_ids is not None:
            if text_stream_ids.dim() == 2 and attention_mask is not None and kw.get("cu_seqlens") is None:
                stream = text_stream_ids[attention_mask.bool()]
            else:
                stream = text_stream_ids.reshape(-1)
        mask = audio_attention_mask if audio_attention_mask is not None else feature_attention_mask
        feats = input_features if input_features is not None and input_features.numel() > 0 else None
        self._rt = (stream, feats, mask, audio_stream_cache)
        try:
            return super().forward(input_ids=input_ids, attention_mask=attention_mask, **kw)
        finally:
            self._rt = None

    # ---- hub names ----------------------------------------------------------------------------
    def convert_hf_state_dict(self, sd):
        out = {}
        for k, v in sd.items():
            if k.startswith("vision_tower."):
                out["visual." + k[len("vision_tower."):]] = v
            elif k.startswith("language_model."):
                out["model.language_model." + k[len("language_model."):]] = v
            else:
                out[k] = v
        return super().convert_hf_state_dict(out)

    def export_hf_state_dict(self, sd):
        out = {}
        for k, v in sd.items():
            if k.startswith("visual."):
                out["vision_tower." + k[len("visual."):]] = v
            elif k.startswith("language_model.model."):
                out["language_model." + k[len("language_model.model."):]] = v
            elif k.startswith("language_model.lm_head."):
                out[k[len("language_model."):]] = v
            else:
                out[k] = v
        return out
