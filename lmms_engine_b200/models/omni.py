"""Qwen2.5-Omni "thinker": the Qwen2.5-VL vision tower and packed decoder plus the chunked audio encoder
(``model_type: qwen2_5_omni_thinker`` / ``qwen2_5_omni``).  The reference patches the ``transformers`` classes
(src/lmms_engine/models/qwen2_5_omni/monkey_patch.py, qwen2_5_omni_ops.py); the talker / token2wav parts of the
hub model are not part of training there and are not built here.

Audio placeholders take the rows of the audio encoder in order; their rotary positions advance by one per
token on all three axes, like text, so the multimodal position builder of the VL models applies unchanged
(videos use ``position_id_per_seconds`` temporal steps).  Hub checkpoints keep separate q / k / v projections
in the vision blocks; they are concatenated into the fused ``qkv`` weight at load time.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict

import torch

from .audio import Omni3AudioEncoder, Omni3AudioEncoderConfig, OmniAudioEncoder, OmniAudioEncoderConfig
from .vl import VLConfig, VLModel


@dataclass
class OmniThinkerConfig(VLConfig):
    audio_config: Any = None
    audio_token_id: int = 151646

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "OmniThinkerConfig":
        d = dict(d.get("thinker_config") or d)  # the full Omni config nests the thinker
        audio = dict(d.pop("audio_config", None) or {})
        ids = {"image_token_id": d.pop("image_token_index", None), "video_token_id": d.pop("video_token_index", None),
               "audio_token_id": d.pop("audio_token_index", None)}
        d.update({k: v for k, v in ids.items() if v is not None and k != "audio_token_id"})
        mt = d.get("model_type", "qwen2_5_omni_thinker")
        vis = dict(d.get("vision_config") or {})
        vis.setdefault("tokens_per_second", int(d.get("position_id_per_seconds", 25)))
        d["vision_config"] = vis
        d["model_type"] = "qwen2_5_vl"  # text / vision defaults of the 2.5 family
        text = dict(d.get("text_config") or {})
        # the thinker's own flag decides (its lm_head is a separate tensor in the hub checkpoints)
        text["tie_word_embeddings"] = bool(d.get("tie_word_embeddings", False))
        d["text_config"] = text
        base = VLConfig.from_dict(d)
        cfg = cls(**{f: getattr(base, f) for f in VLConfig.__dataclass_fields__})
        cfg.model_type = mt
        cfg.extra = {k: v for k, v in base.extra.items() if k not in ("audio_token_id",)}
        audio.setdefault("output_dim", cfg.text_config.hidden_size)
        cfg.audio_config = OmniAudioEncoderConfig.from_dict(audio)
        if ids["audio_token_id"] is not None:
            cfg.audio_token_id = int(ids["audio_token_id"])
        elif "audio_token_id" in base.extra:
            cfg.audio_token_id = int(base.extra["audio_token_id"])
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        d = super().to_dict()
        d["model_type"] = self.model_type
        d["architectures"] = ["Qwen2_5OmniThinkerForConditionalGeneration"]
        d["audio_config"] = {f: getattr(self.audio_config, f) for f in self.audio_config.__dataclass_fields__}
        d["audio_token_index"], d["image_token_index"], d["video_token_index"] = self.audio_token_id, self.image_token_id, self.video_token_id
        return d

    @property
    def is_qwen3(self) -> bool:
        return False


class OmniThinker(VLModel):
    config_class = OmniThinkerConfig
    _no_split_modules = VLModel._no_split_modules + ["AudioEncoderLayer"]

    def __init__(self, cfg: OmniThinkerConfig):
        base = VLConfig(**{f: getattr(cfg, f) for f in VLConfig.__dataclass_fields__})
        base.model_type = "qwen2_5_vl"
        super().__init__(base)
        self.config = cfg
        self.audio_tower = OmniAudioEncoder(cfg.audio_config)

    def embed_multimodal(self, ids, pixel_values, image_grid_thw, pixel_values_videos, video_grid_thw):
        emb, deep, idx = super().embed_multimodal(ids, pixel_values, image_grid_thw, pixel_values_videos, video_grid_thw)
        audio = getattr(self, "_audio_inputs", None)
        if audio is not None:
            feats_in, mask_in = audio
            lens = mask_in.sum(-1).long()
            stream = torch.cat([feats_in[i, :, : int(n)] for i, n in enumerate(lens.tolist())], 1)
            feats, _ = self.audio_tower(stream, lens)
            m = ids == self.config.audio_token_id
            src = (torch.cumsum(m, 0) - 1).clamp(min=0, max=max(feats.shape[0] - 1, 0))
            emb = torch.where(m.unsqueeze(-1), feats.to(emb.dtype).index_select(0, src), emb)
        return emb, deep, idx

    def forward(self, input_features=None, feature_attention_mask=None, audio_values=None, audio_attention_mask=None, **kw):
        feats = input_features if input_features is not None else audio_values
        mask = feature_attention_mask if feature_attention_mask is not None else audio_attention_mask
        self._audio_inputs = (feats, mask) if feats is not None and feats.numel() > 0 else None
        try:
            return super().forward(**kw)
        finally:
            self._audio_inputs = None

    # ---- hub names ----------------------------------------------------------------------------
    def convert_hf_state_dict(self, sd):
        out, qkv = {}, {}
        for k, v in sd.items():
            if k.startswith("thinker."):
                k = k[len("thinker."):]
            elif k.startswith(("talker.", "token2wav.")):
                continue
            if k.startswith("visual.blocks.") and ".attn." in k and k.split(".attn.")[1].split(".")[0] in ("q", "k", "v"):
                head, tail = k.split(".attn.")
                which, kind = tail.split(".")
                qkv.setdefault((head, kind), {})[which] = v
                continue
            out[k] = v
        for (head, kind), parts in qkv.items():
            out[f"{head}.attn.qkv.{kind}"] = torch.cat([parts["q"], parts["k"], parts["v"]], 0)
        return super().convert_hf_state_dict(out)


@dataclass
class Omni3ThinkerConfig(VLConfig):
    """Qwen3-Omni thinker: mixture-of-experts decoder with interleaved M-RoPE, Qwen3-VL style vision tower
    with deepstack, Qwen3-Omni audio encoder (``model_type: qwen3_omni_moe_thinker`` / ``qwen3_omni_moe``)."""

    audio_config: Any = None
    audio_token_id: int = 151675

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "Omni3ThinkerConfig":
        d = dict(d.get("thinker_config") or d)
        audio = dict(d.pop("audio_config", None) or {})
        audio_tok = d.pop("audio_token_id", None)
        mt = d.get("model_type", "qwen3_omni_moe_thinker")
        text = dict(d.get("text_config") or {})
        text["model_type"] = "qwen3_moe"
        text["tie_word_embeddings"] = bool(d.get("tie_word_embeddings", False))
        d["text_config"] = text
        d["model_type"] = "qwen3_vl_moe"
        base = VLConfig.from_dict(d)
        cfg = cls(**{f: getattr(base, f) for f in VLConfig.__dataclass_fields__})
        cfg.model_type = mt
        audio.setdefault("output_dim", cfg.text_config.hidden_size)
        cfg.audio_config = Omni3AudioEncoderConfig.from_dict(audio)
        if audio_tok is not None:
            cfg.audio_token_id = int(audio_tok)
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        d = super().to_dict()
        d["model_type"] = self.model_type
        d["architectures"] = ["Qwen3OmniMoeThinkerForConditionalGeneration"]
        d["audio_config"] = {f: getattr(self.audio_config, f) for f in self.audio_config.__dataclass_fields__}
        d["audio_token_id"] = self.audio_token_id
        return d

    @property
    def is_qwen3(self) -> bool:
        return True


class Omni3Thinker(OmniThinker):
    config_class = Omni3ThinkerConfig

    def __init__(self, cfg: Omni3ThinkerConfig):
        base = VLConfig(**{f: getattr(cfg, f) for f in VLConfig.__dataclass_fields__})
        base.model_type = "qwen3_vl_moe"
        VLModel.__init__(self, base)
        self.config = cfg
        self.audio_tower = Omni3AudioEncoder(cfg.audio_config)

    def convert_hf_state_dict(self, sd):
        # the hub names of the patch mergers differ from the Qwen3-VL ones that the tower uses
        ren = {}
        for k, v in sd.items():
            k2 = k[len("thinker."):] if k.startswith("thinker.") else k
            if k2.startswith("visual.merger_list."):
                k2 = "visual.deepstack_merger_list." + k2[len("visual.merger_list."):]
            if k2.startswith(("visual.merger.", "visual.deepstack_merger_list.")):
                k2 = k2.replace(".ln_q.", ".norm.").replace(".mlp.0.", ".linear_fc1.").replace(".mlp.2.", ".linear_fc2.")
            ren[k2] = v
        return super().convert_hf_state_dict(ren)
