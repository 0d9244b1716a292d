"""Audio-language model: a Whisper-style mel encoder, a linear projector and a packed decoder
(``model_type: qwen2_audio``).  The reference patches the ``transformers`` classes
(src/lmms_engine/models/qwen2_audio/monkey_patch.py, qwen2_audio_ops.py: varlen attention in the audio
encoder); here the encoder runs natively on the valid frames only.

Module and parameter names follow the hub checkpoints (``audio_tower.*``, ``multi_modal_projector.linear``,
``language_model.*``), so ``hf_io`` loads them without a name map.

Shapes: ``input_features [n_audio, mel_bins, T_mel]`` (padded log-mel), ``feature_attention_mask
[n_audio, T_mel]``.  After the two convolutions (the second with stride 2) an audio of ``L`` mel frames has
``(L - 1) // 2 + 1`` frames; attention runs over exactly those (keys of the padding never take part, as
with the reference's mask); average pooling by 2 leaves ``(frames - 2) // 2 + 1`` feature rows, which
replace the audio placeholder tokens of the stream in order.
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
from .decoder_lm import DecoderConfig, DecoderLM, unpad_batch
from .vision import LayerNorm


@dataclass
class AudioEncoderConfig:
    num_mel_bins: int = 128
    d_model: int = 1280
    encoder_layers: int = 32
    encoder_attention_heads: int = 20
    encoder_ffn_dim: int = 5120
    max_source_positions: int = 1500
    activation_function: str = "gelu"

    @classmethod
    def from_dict(cls, d):
        known = {f.name for f in fields(cls)}
        return cls(**{k: v for k, v in (d or {}).items() if k in known})


@dataclass
class Qwen2AudioConfig:
    model_type: str = "qwen2_audio"
    text_config: Any = None
    audio_config: Any = None
    audio_token_index: int = 151646
    extra: Dict[str, Any] = field(default_factory=dict)

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "Qwen2AudioConfig":
        d = dict(d)
        text, audio = d.pop("text_config", None) or {}, d.pop("audio_config", None) or {}
        known = {f.name for f in fields(cls)}
        kw = {k: v for k, v in d.items() if k in known}
        kw["extra"] = {k: v for k, v in d.items() if k not in known}
        cfg = cls(**kw)
        cfg.text_config = text if isinstance(text, DecoderConfig) else DecoderConfig.from_dict({"model_type": "qwen2", **text})
        cfg.audio_config = audio if isinstance(audio, AudioEncoderConfig) else AudioEncoderConfig.from_dict(audio)
        return cfg

    def to_dict(self):
        return {"model_type": self.model_type, "text_config": self.text_config.to_dict(),
                "audio_config": {f.name: getattr(self.audio_config, f.name) for f in fields(self.audio_config)},
                "audio_token_index": self.audio_token_index, **self.extra}

    @property
    def vocab_size(self):
        return self.text_config.vocab_size


class _SelfAttn(nn.Module):
    def __init__(self, d: int, heads: int):
        super().__init__()
        self.heads, self.head_dim = heads, d // heads
        self.k_proj = nn.Linear(d, d, bias=False)
        self.v_proj = nn.Linear(d, d, bias=True)
        self.q_proj = nn.Linear(d, d, bias=True)
        self.out_proj = nn.Linear(d, d, bias=True)

    def forward(self, x, cu):
        P = x.shape[0]
        w = torch.cat([self.q_proj.weight, self.k_proj.weight, self.v_proj.weight], 0)
        b = torch.cat([self.q_proj.bias, torch.zeros_like(self.q_proj.bias), self.v_proj.bias], 0)
        qkv = gemm_ops.linear(x, w, b).view(P, 3, self.heads, self.head_dim)
        o = attn_ops.varlen_attn(qkv[:, 0], qkv[:, 1], qkv[:, 2], cu, cu, causal=False, softmax_scale=self.head_dim ** -0.5)
        return gemm_ops.linear(o.reshape(P, -1), self.out_proj.weight, self.out_proj.bias)


class AudioEncoderLayer(nn.Module):
    def __init__(self, c: AudioEncoderConfig):
        super().__init__()
        self.self_attn = _SelfAttn(c.d_model, c.encoder_attention_heads)
        self.self_attn_layer_norm = LayerNorm(c.d_model, 1e-5)
        self.fc1, self.fc2 = nn.Linear(c.d_model, c.encoder_ffn_dim), nn.Linear(c.encoder_ffn_dim, c.d_model)
        self.final_layer_norm = LayerNorm(c.d_model, 1e-5)

    def forward(self, x, cu):
        x = x + self.self_attn(self.self_attn_layer_norm(x), cu)
        h = F.gelu(gemm_ops.linear(self.final_layer_norm(x), self.fc1.weight, self.fc1.bias))
        return x + gemm_ops.linear(h, self.fc2.weight, self.fc2.bias)


class AudioEncoder(nn.Module):
    def __init__(self, c: AudioEncoderConfig):
        super().__init__()
        self.cfg = c
        self.conv1 = nn.Conv1d(c.num_mel_bins, c.d_model, kernel_size=3, padding=1)
        self.conv2 = nn.Conv1d(c.d_model, c.d_model, kernel_size=3, stride=2, padding=1)
        self.embed_positions = nn.Embedding(c.max_source_positions, c.d_model)
        self.embed_positions.requires_grad_(False)
        self.layers = nn.ModuleList([AudioEncoderLayer(c) for _ in range(c.encoder_layers)])
        self.layer_norm = LayerNorm(c.d_model, 1e-5)

    @staticmethod
    def output_lengths(mel_lengths: torch.Tensor):
        frames = (mel_lengths - 1) // 2 + 1
        return frames, (frames - 2) // 2 + 1

    def forward(self, input_features: torch.Tensor, feature_attention_mask: torch.Tensor):
        """Returns the pooled features of all audios concatenated, ``[sum(out_len), d_model]``, and ``out_len``."""
        x = F.gelu(self.conv1(input_features.to(self.conv1.weight.dtype)))
        x = F.gelu(self.conv2(x)).permute(0, 2, 1)  # [n, frames_max, d]
        x = x + self.embed_positions.weight[: x.shape[1]].to(x.dtype)
        frames, out_len = self.output_lengths(feature_attention_mask.sum(-1).long())
        fr = frames.tolist()
        flat = torch.cat([x[i, :n] for i, n in enumerate(fr)], 0)  # valid frames only
        cu = torch.cumsum(torch.tensor([0] + fr, device=x.device), 0).to(torch.int32)
        for layer in self.layers:
            flat = layer(flat, cu)
        pooled, start = [], 0
        for n, m in zip(fr, out_len.tolist()):
            seg = flat[start:start + 2 * m].view(m, 2, -1).mean(1) if m > 0 else flat[:0]
            pooled.append(seg)
            start += n
        return self.layer_norm(torch.cat(pooled, 0)), out_len


class _Projector(nn.Module):
    def __init__(self, d_in: int, d_out: int):
        super().__init__()
        self.linear = nn.Linear(d_in, d_out, bias=True)

    def forward(self, x):
        return gemm_ops.linear(x, self.linear.weight, self.linear.bias)


class Qwen2AudioModel(nn.Module):
    config_class = Qwen2AudioConfig
    _no_split_modules = ["DecoderLayer", "AudioEncoderLayer"]
    projector_name = "multi_modal_projector"  # parameter prefix of the projector in hub checkpoints

    def __init__(self, cfg: Qwen2AudioConfig):
        super().__init__()
        self.config = cfg
        self.audio_tower = AudioEncoder(cfg.audio_config)
        setattr(self, self.projector_name, _Projector(cfg.audio_config.d_model, cfg.text_config.hidden_size))
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

    def forward(self, input_ids=None, labels=None, attention_mask=None, input_features=None, feature_attention_mask=None,
                audio_values=None, audio_attention_mask=None, cu_seqlens=None, position_ids=None, **kw):
        ids, lab, cu, pos = input_ids, labels, cu_seqlens, position_ids
        if ids.dim() == 2:
            ids, lab, pos, cu, _ = unpad_batch(ids, attention_mask if attention_mask is not None else torch.ones_like(ids), lab)
        else:
            ids, lab, pos, cu, _ = self.language_model.prepare_packed(ids, None, lab, pos, cu)
        emb = self.get_input_embeddings()(ids)
        feats_in = input_features if input_features is not None else audio_values
        mask_in = feature_attention_mask if feature_attention_mask is not None else audio_attention_mask
        if feats_in is not None and feats_in.numel() > 0:
            feats, _ = self.audio_tower(feats_in, mask_in)
            feats = getattr(self, self.projector_name)(feats).to(emb.dtype)
            m = ids == self.config.audio_token_index
            src = (torch.cumsum(m, 0) - 1).clamp(min=0, max=max(feats.shape[0] - 1, 0))
            emb = torch.where(m.unsqueeze(-1), feats.index_select(0, src), emb)
        return self.language_model(inputs_embeds=emb, labels=lab, cu_seqlens=cu, position_ids=pos)


@dataclass
class AeroConfig(Qwen2AudioConfig):
    """``model_type: aero`` with the Qwen2-Audio encoder (reference: src/lmms_engine/models/aero/configuration_aero.py:28-66;
    its Qwen2.5-Omni encoder option is not built)."""

    model_type: str = "aero"
    audio_token_index: int = 151648


class AeroModel(Qwen2AudioModel):
    """Audio-LM of the reference (src/lmms_engine/models/aero/modeling_aero.py:230-420): same structure as
    Qwen2-Audio, projector stored as ``audio_modal_projector``."""

    config_class = AeroConfig
    projector_name = "audio_modal_projector"
