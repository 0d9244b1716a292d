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
from typing import Any, Dict, List, Optional

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
class OmniAudioEncoderConfig(AudioEncoderConfig):
    n_window: int = 100
    output_dim: int = 3584


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
        if isinstance(audio, AudioEncoderConfig):
            cfg.audio_config = audio
        elif audio.get("model_type") == "qwen2_5_omni_audio_encoder":
            cfg.audio_config = OmniAudioEncoderConfig.from_dict(audio)
        else:
            cfg.audio_config = AudioEncoderConfig.from_dict(audio)
        return cfg

    def to_dict(self):
        return {"model_type": self.model_type, "text_config": self.text_config.to_dict(),
                "audio_config": {"model_type": ("qwen2_5_omni_audio_encoder" if isinstance(self.audio_config, OmniAudioEncoderConfig)
                                                else "qwen2_audio_encoder"),
                                 **{f.name: getattr(self.audio_config, f.name) for f in fields(self.audio_config)}},
                "audio_token_index": self.audio_token_index, **self.extra}

    @property
    def vocab_size(self):
        return self.text_config.vocab_size


class _SelfAttn(nn.Module):
    def __init__(self, d: int, heads: int, k_bias: bool = False):
        super().__init__()
        self.heads, self.head_dim = heads, d // heads
        self.k_proj = nn.Linear(d, d, bias=k_bias)
        self.v_proj = nn.Linear(d, d, bias=True)
        self.q_proj = nn.Linear(d, d, bias=True)
        self.out_proj = nn.Linear(d, d, bias=True)

    def forward(self, x, cu):
        P = x.shape[0]
        w = torch.cat([self.q_proj.weight, self.k_proj.weight, self.v_proj.weight], 0)
        kb = self.k_proj.bias if self.k_proj.bias is not None else torch.zeros_like(self.q_proj.bias)
        b = torch.cat([self.q_proj.bias, kb, self.v_proj.bias], 0)
        qkv = gemm_ops.linear(x, w, b).view(P, 3, self.heads, self.head_dim)
        o = attn_ops.varlen_attn(qkv[:, 0], qkv[:, 1], qkv[:, 2], cu, cu, causal=False, softmax_scale=self.head_dim ** -0.5)
        return gemm_ops.linear(o.reshape(P, -1), self.out_proj.weight, self.out_proj.bias)


class AudioEncoderLayer(nn.Module):
    def __init__(self, c: AudioEncoderConfig, k_bias: bool = False):
        super().__init__()
        self.self_attn = _SelfAttn(c.d_model, c.encoder_attention_heads, k_bias)
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


class OmniAudioEncoder(nn.Module):
    """Audio encoder of Qwen2.5-Omni (also an option of ``aero``): the mel stream is cut into chunks of
    ``2 * n_window`` frames, attention stays inside a chunk (one varlen document per chunk, sinusoidal
    positions restart per chunk), features are average-pooled by 2 per clip and projected to ``output_dim``.
    Input: ``input_features [mel_bins, sum(feature_lens)]`` (clips concatenated in time), ``feature_lens``."""

    def __init__(self, c: OmniAudioEncoderConfig):
        super().__init__()
        self.cfg = c
        self.n_window = c.n_window
        self.conv1 = nn.Conv1d(c.num_mel_bins, c.d_model, kernel_size=3, padding=1)
        self.conv2 = nn.Conv1d(c.d_model, c.d_model, kernel_size=3, stride=2, padding=1)
        half = c.d_model // 2
        inv = torch.exp(-(math.log(10000.0) / (half - 1)) * torch.arange(half).float())
        t = torch.arange(c.max_source_positions)[:, None] * inv[None, :]
        self.register_buffer("positional_embedding", torch.cat([torch.sin(t), torch.cos(t)], 1), persistent=False)
        self.audio_bos_eos_token = nn.Embedding(2, c.output_dim)
        self.layers = nn.ModuleList([AudioEncoderLayer(c) for _ in range(c.encoder_layers)])
        self.ln_post = LayerNorm(c.d_model, 1e-5)
        self.proj = nn.Linear(c.d_model, c.output_dim)

    @staticmethod
    def output_lengths(feature_lens: torch.Tensor):
        after_cnn = (feature_lens - 1) // 2 + 1
        return after_cnn, (after_cnn - 2) // 2 + 1

    def forward(self, input_features: torch.Tensor, feature_lens: torch.Tensor):
        w2 = self.n_window * 2
        lens = feature_lens.tolist()
        chunk_lengths = []
        for L in lens:
            n = -(-L // w2)
            chunk_lengths += [w2] * (n - 1) + [L - (n - 1) * w2]
        dt = self.conv1.weight.dtype
        chunks = input_features.to(dt).split(chunk_lengths, dim=1)
        max_len = max(chunk_lengths)
        padded = input_features.new_zeros((len(chunks), input_features.shape[0], max_len), dtype=dt)
        mask = torch.zeros((len(chunks), 1, max_len), dtype=dt, device=input_features.device)
        for i, (ch, L) in enumerate(zip(chunks, chunk_lengths)):
            padded[i, :, :L] = ch
            mask[i, 0, :L] = 1
        x = F.gelu(self.conv1(padded)) * mask
        x = F.gelu(self.conv2(x)).transpose(1, 2)
        x = x + self.positional_embedding[: x.shape[1]].to(x.dtype)
        after = [(L - 1) // 2 + 1 for L in chunk_lengths]
        flat = torch.cat([x[i, :n] for i, n in enumerate(after)], 0)
        cu = torch.cumsum(torch.tensor([0] + after, device=x.device), 0).to(torch.int32)
        for layer in self.layers:
            flat = layer(flat, cu)
        after_cnn, out_len = self.output_lengths(feature_lens)
        outs, start = [], 0
        for n, m in zip(after_cnn.tolist(), out_len.tolist()):
            seg = flat[start:start + 2 * m].view(m, 2, -1).mean(1) if m > 0 else flat[:0]
            outs.append(seg)
            start += n
        h = self.ln_post(torch.cat(outs, 0))
        return gemm_ops.linear(h, self.proj.weight, self.proj.bias), out_len


@dataclass
class Omni3AudioEncoderConfig(OmniAudioEncoderConfig):
    n_window: int = 50
    n_window_infer: int = 400
    downsample_hidden_size: int = 480
    conv_chunksize: int = 500


def omni3_output_lengths(input_lengths: torch.Tensor) -> torch.Tensor:
    """Rows the Qwen3-Omni encoder emits for ``input_lengths`` mel frames (three stride-2 convolutions per
    100-frame chunk: 13 rows per full chunk)."""
    leave = input_lengths % 100
    feat = (leave - 1) // 2 + 1
    return ((feat - 1) // 2 + 1 - 1) // 2 + 1 + (input_lengths // 100) * 13


class Omni3AudioEncoder(nn.Module):
    """Audio encoder of Qwen3-Omni: chunks of ``2 * n_window`` mel frames go through three stride-2 2-D
    convolutions (time and frequency) and a linear layer, attention runs inside windows of
    ``n_window_infer / (2 * n_window)`` chunks (one varlen document per window), then LayerNorm and a
    two-layer projection to ``output_dim``.  Input as for ``OmniAudioEncoder``."""

    def __init__(self, c: Omni3AudioEncoderConfig):
        super().__init__()
        self.cfg = c
        self.n_window, self.n_window_infer, self.conv_chunksize = c.n_window, c.n_window_infer, c.conv_chunksize
        half = c.d_model // 2
        inv = torch.exp(-(math.log(10000.0) / (half - 1)) * torch.arange(half).float())
        t = torch.arange(c.max_source_positions)[:, None] * inv[None, :]
        self.register_buffer("positional_embedding", torch.cat([torch.sin(t), torch.cos(t)], 1), persistent=False)
        self.layers = nn.ModuleList([AudioEncoderLayer(c, k_bias=True) for _ in range(c.encoder_layers)])
        self.ln_post = LayerNorm(c.d_model, 1e-5)
        h = c.downsample_hidden_size
        self.conv2d1 = nn.Conv2d(1, h, 3, 2, padding=1)
        self.conv2d2 = nn.Conv2d(h, h, 3, 2, padding=1)
        self.conv2d3 = nn.Conv2d(h, h, 3, 2, padding=1)
        self.conv_out = nn.Linear(h * ((((c.num_mel_bins + 1) // 2 + 1) // 2 + 1) // 2), c.d_model, bias=False)
        self.proj1 = nn.Linear(c.d_model, c.d_model)
        self.proj2 = nn.Linear(c.d_model, c.output_dim)

    def forward(self, input_features: torch.Tensor, feature_lens: torch.Tensor):
        w2 = self.n_window * 2
        lens = feature_lens.tolist()
        chunk_lengths = []
        for L in lens:
            n = -(-L // w2)
            chunk_lengths += [w2] * (n - 1) + [L - (n - 1) * w2]
        dt = self.conv2d1.weight.dtype
        chunks = input_features.to(dt).T.split(chunk_lengths, dim=0)
        padded = nn.utils.rnn.pad_sequence(chunks, batch_first=True).transpose(1, 2).unsqueeze(1)  # [n, 1, mel, t]
        after = omni3_output_lengths(torch.tensor(chunk_lengths)).tolist()
        embeds = []
        for part in padded.split(self.conv_chunksize, dim=0):
            e = F.gelu(self.conv2d1(part))
            e = F.gelu(self.conv2d2(e))
            embeds.append(F.gelu(self.conv2d3(e)))
        e = torch.cat(embeds, 0)
        b, c, f, t = e.shape
        x = gemm_ops.linear(e.permute(0, 3, 1, 2).reshape(b * t, c * f), self.conv_out.weight, None).view(b, t, -1)
        x = x + self.positional_embedding[:t].to(x.dtype)
        flat = torch.cat([x[i, :n] for i, n in enumerate(after)], 0)
        out_len = omni3_output_lengths(feature_lens)
        window = max(after) * (self.n_window_infer // w2)
        pieces = [0]
        for n in out_len.tolist():
            pieces += [window] * (n // window) + ([n % window] if n % window else [])
        cu = torch.cumsum(torch.tensor(pieces, device=x.device), 0).to(torch.int32)
        for layer in self.layers:
            flat = layer(flat, cu)
        h = F.gelu(gemm_ops.linear(self.ln_post(flat), self.proj1.weight, self.proj1.bias))
        return gemm_ops.linear(h, self.proj2.weight, self.proj2.bias), out_len


class _Projector(nn.Module):
    def __init__(self, d_in: int, d_out: int, pre_gelu: bool = False):
        super().__init__()
        self.linear = nn.Linear(d_in, d_out, bias=True)
        self.pre_gelu = pre_gelu

    def forward(self, x):
        return gemm_ops.linear(F.gelu(x) if self.pre_gelu else x, self.linear.weight, self.linear.bias)


class Qwen2AudioModel(nn.Module):
    config_class = Qwen2AudioConfig
    _no_split_modules = ["DecoderLayer", "AudioEncoderLayer"]
    projector_name = "multi_modal_projector"  # parameter prefix of the projector in hub checkpoints

    def __init__(self, cfg: Qwen2AudioConfig):
        super().__init__()
        self.config = cfg
        self.omni_encoder = isinstance(cfg.audio_config, OmniAudioEncoderConfig)
        if self.omni_encoder:
            self.audio_tower = OmniAudioEncoder(cfg.audio_config)
            proj = _Projector(cfg.audio_config.output_dim, cfg.text_config.hidden_size, pre_gelu=True)
        else:
            self.audio_tower = AudioEncoder(cfg.audio_config)
            proj = _Projector(cfg.audio_config.d_model, cfg.text_config.hidden_size)
        setattr(self, self.projector_name, proj)
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
            if self.omni_encoder:
                # clips concatenated in time, valid frames only
                lens = mask_in.sum(-1).long()
                stream = torch.cat([feats_in[i, :, : int(n)] for i, n in enumerate(lens.tolist())], 1)
                feats, _ = self.audio_tower(stream, lens)
            else:
                feats, _ = self.audio_tower(feats_in, mask_in)
            feats = getattr(self, self.projector_name)(feats).to(emb.dtype)
            m = ids == self.config.audio_token_index
            src = (torch.cumsum(m, 0) - 1).clamp(min=0, max=max(feats.shape[0] - 1, 0))
            emb = torch.where(m.unsqueeze(-1), feats.index_select(0, src), emb)
        return self.language_model(inputs_embeds=emb, labels=lab, cu_seqlens=cu, position_ids=pos)


@dataclass
class AeroConfig(Qwen2AudioConfig):
    """``model_type: aero`` (reference: src/lmms_engine/models/aero/configuration_aero.py:28-66); ``audio_config.model_type``
    selects the Qwen2-Audio encoder (default) or the chunked Qwen2.5-Omni encoder."""

    model_type: str = "aero"
    audio_token_index: int = 151648


class AeroModel(Qwen2AudioModel):
    """Audio-LM of the reference (src/lmms_engine/models/aero/modeling_aero.py:230-420): same structure as
    Qwen2-Audio, projector stored as ``audio_modal_projector``."""

    config_class = AeroConfig
    projector_name = "audio_modal_projector"


# ------------------------------------------------------------------------------- streaming (causal) encoder
@dataclass
class VoxtralRealtimeEncoderConfig:
    model_type: str = "voxtral_realtime_encoder"
    hidden_size: int = 1280
    intermediate_size: int = 5120
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    head_dim: int = 64
    num_mel_bins: int = 128
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    sliding_window: Optional[int] = 750
    max_position_embeddings: int = 1500
    # variants of the realtime model's own encoder (src/lmms_engine/models/aero_realtime/configuration_aero_realtime.py:41-114);
    # the defaults are the released streaming encoder
    norm_type: str = "rms_norm"            # rms_norm | layer_norm
    mlp_type: str = "swiglu"               # swiglu | gelu (fc1 / fc2 with biases)
    conv_padding: str = "causal"           # causal | symmetric (every chunk is encoded by itself)
    activation_function: str = "gelu"
    attention_window_left: Optional[int] = None   # None: sliding_window - 1 (or unlimited); negative: unlimited
    attention_window_right: int = 0                # 0: causal; n > 0: a frame also sees the next n; negative: all that follow
    extra: Dict[str, Any] = field(default_factory=dict)

    def __post_init__(self):
        if self.norm_type not in ("rms_norm", "layer_norm"):
            raise ValueError(f"norm_type must be 'rms_norm' or 'layer_norm', got {self.norm_type}")
        if self.mlp_type not in ("swiglu", "gelu"):
            raise ValueError(f"mlp_type must be 'swiglu' or 'gelu', got {self.mlp_type}")
        if self.conv_padding not in ("causal", "symmetric"):
            raise ValueError(f"conv_padding must be 'causal' or 'symmetric', got {self.conv_padding}")
        if self.attention_window_left is None:
            self.attention_window_left = (self.sliding_window - 1) if self.sliding_window else -1

    @classmethod
    def from_dict(cls, d):
        d = dict(d)
        rp = d.get("rope_parameters") or {}
        if "rope_theta" in rp:
            d.setdefault("rope_theta", rp["rope_theta"])
        known = {f.name for f in fields(cls)}
        kw = {k: v for k, v in d.items() if k in known}
        kw["extra"] = {k: v for k, v in d.items() if k not in known}
        return cls(**kw)

    def to_dict(self):
        d = {f.name: getattr(self, f.name) for f in fields(self) if f.name != "extra"}
        d.update(self.extra)
        return d


class _CausalConv1d(nn.Conv1d):
    """Left-padded so that frame t never sees later frames (kernel 3: pad 2 at stride 1, pad 1 at stride 2); with
    ``symmetric = True`` the same total padding is split between both ends (the left half rounded down), which gives the
    same number of frames and lets a chunk be encoded without its neighbours."""

    symmetric = False

    def forward(self, x):
        k = (self.kernel_size[0] - 1) * self.dilation[0] + 1
        total = k - self.stride[0]
        left = total // 2 if self.symmetric else total
        return super().forward(F.pad(x, (left, total - left)))


    def left_pad(self) -> int:
        return (self.kernel_size[0] - 1) * self.dilation[0] + 1 - self.stride[0]

    def continue_from(self, x, tail):
        """The convolution of a stream that arrives in pieces: ``tail`` holds the last ``left_pad`` input frames of what
        came before (zeros at the start, which is the padding of the one-piece form).  Returns the output frames of this
        piece and the tail for the next one.  A piece must hold a whole number of strides."""
        if x.shape[-1] % self.stride[0]:
            raise ValueError(f"a piece of {x.shape[-1]} frames is not a multiple of the stride {self.stride[0]}")
        full = torch.cat([tail.to(x.dtype), x], -1)
        return nn.Conv1d.forward(self, full), full[..., full.shape[-1] - self.left_pad():]


class _VoxtralEmbedder(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.conv1 = _CausalConv1d(c.num_mel_bins, c.hidden_size, kernel_size=3)
        self.conv2 = _CausalConv1d(c.hidden_size, c.hidden_size, kernel_size=3, stride=2)
        self.conv1.symmetric = self.conv2.symmetric = getattr(c, "conv_padding", "causal") == "symmetric"


def local_window_attention(q, k, v, cu, left: int, right: int, scale: float):
    """Attention of packed documents in which frame i sees frames ``i - left .. i + right`` (a negative bound is no bound).
    The dense form of the masks the varlen kernel does not cover - a bounded look-ahead, or a left bound without
    causality (src/lmms_engine/models/aero_realtime/modeling_aero_realtime.py:914-935); the audio encoder's documents are
    a few thousand frames at most.  ``q / k / v [P, heads, head_dim]``."""
    out = torch.empty_like(q)
    bounds = cu.tolist()
    for a, b in zip(bounds[:-1], bounds[1:]):
        i = torch.arange(b - a, device=q.device)
        delta = i[None, :] - i[:, None]
        allow = torch.ones_like(delta, dtype=torch.bool)
        if left >= 0:
            allow &= delta >= -left
        if right >= 0:
            allow &= delta <= right
        o = F.scaled_dot_product_attention(q[a:b].transpose(0, 1), k[a:b].transpose(0, 1), v[a:b].transpose(0, 1), attn_mask=allow, scale=scale)
        out[a:b] = o.transpose(0, 1)
    return out


class _VoxtralAttention(nn.Module):
    def __init__(self, c):
        super().__init__()
        d, hd = c.hidden_size, c.head_dim
        self.heads, self.head_dim = c.num_attention_heads, hd
        self.q_proj = nn.Linear(d, self.heads * hd, bias=True)
        self.k_proj = nn.Linear(d, self.heads * hd, bias=False)
        self.v_proj = nn.Linear(d, self.heads * hd, bias=True)
        self.o_proj = nn.Linear(self.heads * hd, d, bias=True)
        left = getattr(c, "attention_window_left", None)
        left = ((c.sliding_window - 1) if c.sliding_window else -1) if left is None else left
        right = getattr(c, "attention_window_right", 0)
        self.causal = right == 0
        self.left, self.right = (left if left >= 0 else -1), (right if right >= 0 else -1)
        # the varlen kernel covers causal masks (with or without a left bound) and the full mask
        self.kernel_mask = self.causal or (self.left < 0 and self.right < 0)
        self.window = (left, -1) if left >= 0 else (-1, -1)

    def forward(self, x, cu, cos, sin, past=None):
        """``past``: ``None``, or a two-entry list ``[keys, values]`` of the frames that came before (rotated keys), which
        is extended in place by this piece and trimmed to the left window: the streaming form, causal masks only."""
        from ..ops import rope as rope_ops

        P = x.shape[0]
        w = torch.cat([self.q_proj.weight, self.k_proj.weight, self.v_proj.weight], 0)
        b = torch.cat([self.q_proj.bias, torch.zeros_like(self.q_proj.bias), self.v_proj.bias], 0)
        qkv = gemm_ops.linear(x, w, b).view(P, 3, self.heads, self.head_dim)
        q, k = rope_ops.rope_apply(qkv[:, 0], cos, sin), rope_ops.rope_apply(qkv[:, 1], cos, sin)
        v = qkv[:, 2]
        scale = self.head_dim ** -0.5
        if past is not None:
            if not self.causal:
                raise ValueError("an encoder whose frames see what follows cannot run on a stream")
            if past[0] is not None:
                k, v = torch.cat([past[0], k], 0), torch.cat([past[1], v], 0)
            keep = k.shape[0] if self.left < 0 else min(k.shape[0], self.left)
            past[0], past[1] = k[k.shape[0] - keep:].detach(), v[v.shape[0] - keep:].detach()
            cu_k = torch.tensor([0, k.shape[0]], dtype=torch.int32, device=x.device)
            o = attn_ops.varlen_attn(q, k.contiguous(), v.contiguous(), cu, cu_k, causal=True, softmax_scale=scale, window_size=self.window)
        elif self.kernel_mask:
            o = attn_ops.varlen_attn(q, k, v, cu, cu, causal=self.causal, softmax_scale=scale, window_size=self.window)
        else:
            o = local_window_attention(q, k, v, cu, self.left, self.right, scale)
        return gemm_ops.linear(o.reshape(P, -1), self.o_proj.weight, self.o_proj.bias)


class _VoxtralMLP(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.gate_proj = nn.Linear(c.hidden_size, c.intermediate_size, bias=False)
        self.up_proj = nn.Linear(c.hidden_size, c.intermediate_size, bias=False)
        self.down_proj = nn.Linear(c.intermediate_size, c.hidden_size, bias=True)

    def forward(self, x):
        from ..ops import swiglu as swiglu_ops

        h = swiglu_ops.swiglu(gemm_ops.linear(x, self.gate_proj.weight, None), gemm_ops.linear(x, self.up_proj.weight, None))
        return gemm_ops.linear(h, self.down_proj.weight, self.down_proj.bias)


class _VoxtralGeluMLP(nn.Module):
    """``fc2(act(fc1(x)))`` with biases: the ``mlp_type: gelu`` variant."""

    def __init__(self, c):
        super().__init__()
        self.fc1 = nn.Linear(c.hidden_size, c.intermediate_size)
        self.fc2 = nn.Linear(c.intermediate_size, c.hidden_size)
        self.act = getattr(c, "activation_function", "gelu")

    def forward(self, x):
        h = gemm_ops.linear(x, self.fc1.weight, self.fc1.bias)
        h = F.silu(h) if self.act in ("silu", "swish") else F.gelu(h, approximate="tanh" if "tanh" in self.act or self.act == "gelu_new" else "none")
        return gemm_ops.linear(h, self.fc2.weight, self.fc2.bias)


def _encoder_norm(c):
    from .decoder_lm import RMSNorm

    if getattr(c, "norm_type", "rms_norm") == "layer_norm":
        return nn.LayerNorm(c.hidden_size, eps=c.rms_norm_eps)
    return RMSNorm(c.hidden_size, c.rms_norm_eps)


class VoxtralEncoderLayer(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.self_attn = _VoxtralAttention(c)
        self.self_attn_layer_norm, self.final_layer_norm = _encoder_norm(c), _encoder_norm(c)
        self.mlp = _VoxtralGeluMLP(c) if getattr(c, "mlp_type", "swiglu") == "gelu" else _VoxtralMLP(c)

    def forward(self, x, cu, cos, sin, past=None):
        x = x + self.self_attn(self.self_attn_layer_norm(x), cu, cos, sin, past)
        return x + self.mlp(self.final_layer_norm(x))


class VoxtralStreamCache:
    """What the streaming encoder carries from one piece of a clip to the next: the last input frames of both
    convolutions (the reference's padding cache, src/lmms_engine/models/aero_realtime/modeling_aero_realtime.py:678-736),
    every layer's rotated keys and values inside the left window, and the number of frames encoded so far (the rotary
    position of the next one)."""

    def __init__(self, n_layers: int):
        self.conv_tails: List[Optional[torch.Tensor]] = [None, None]
        self.layers: List[List[Optional[torch.Tensor]]] = [[None, None] for _ in range(n_layers)]
        self.frames = 0


class VoxtralRealtimeEncoder(nn.Module):
    """Streaming audio encoder (reference: src/lmms_engine/models/voxtral_realtime/voxtral_realtime_ops.py, a patch of the
    ``transformers`` class): causal convolutions, rotary causal attention inside a sliding window, RMSNorm, gated MLP.
    ``input_features [n, mel, T]`` with ``feature_attention_mask [n, T]`` (or full clips); every clip is one varlen
    document of ``floor(L / 2)`` frames.  Returns ``{"last_hidden_state": [sum(frames), hidden], "frame_lengths"}``."""

    config_class = VoxtralRealtimeEncoderConfig
    _no_split_modules = ["VoxtralEncoderLayer"]

    def __init__(self, c: VoxtralRealtimeEncoderConfig):
        super().__init__()
        from .decoder_lm import RMSNorm

        self.config = c
        self.embedder = _VoxtralEmbedder(c)
        self.layers = nn.ModuleList([VoxtralEncoderLayer(c) for _ in range(c.num_hidden_layers)])
        self.norm = _encoder_norm(c)

    def forward(self, input_features, feature_attention_mask=None, **kw):
        n, _, T = input_features.shape
        lens = feature_attention_mask.sum(-1).long() if feature_attention_mask is not None else torch.full((n,), T, device=input_features.device)
        x = F.gelu(self.embedder.conv1(input_features.to(self.embedder.conv1.weight.dtype)))
        x = F.gelu(self.embedder.conv2(x)).permute(0, 2, 1)  # causal: frame j covers mel frames <= 2j+1
        frames = (lens // 2).clamp(min=1).tolist()  # the stride-2 causal convolution yields floor(L / 2) frames
        flat = torch.cat([x[i, :f] for i, f in enumerate(frames)], 0)
        cu = torch.cumsum(torch.tensor([0] + frames, device=x.device), 0).to(torch.int32)
        pos = torch.cat([torch.arange(f, device=x.device) for f in frames]).float()
        hd = self.config.head_dim
        inv = 1.0 / (self.config.rope_theta ** (torch.arange(0, hd, 2, device=x.device).float() / hd))
        ang = pos[:, None] * inv[None, :]
        cos, sin = torch.cat([ang.cos(), ang.cos()], -1), torch.cat([ang.sin(), ang.sin()], -1)
        for layer in self.layers:
            flat = layer(flat, cu, cos, sin)
        return {"last_hidden_state": self.norm(flat), "frame_lengths": torch.tensor(frames, device=x.device)}

    def _rotary(self, pos):
        hd = self.config.head_dim
        inv = 1.0 / (self.config.rope_theta ** (torch.arange(0, hd, 2, device=pos.device).float() / hd))
        ang = pos[:, None] * inv[None, :]
        return torch.cat([ang.cos(), ang.cos()], -1), torch.cat([ang.sin(), ang.sin()], -1)

    def new_stream(self) -> VoxtralStreamCache:
        c = self.config
        if getattr(c, "conv_padding", "causal") != "causal" or getattr(c, "attention_window_right", 0) != 0:
            raise ValueError("only the causal encoder (causal convolution padding, no look-ahead) encodes a stream piece by piece; "
                             "the other variants encode every chunk by itself")
        return VoxtralStreamCache(len(self.layers))

    def stream(self, piece: torch.Tensor, cache: VoxtralStreamCache) -> torch.Tensor:
        """Encode the next ``piece [mel, 2 m]`` (an even number of mel frames) of ONE clip and return its ``m`` frames
        ``[m, hidden]``: the same rows the one-piece ``forward`` gives for these frames, because the convolutions continue
        from the cached input tails and attention runs against the cached keys of the left window."""
        x = piece.reshape(1, piece.shape[-2], piece.shape[-1]).to(self.embedder.conv1.weight.dtype)
        e = self.embedder
        tails = cache.conv_tails
        if tails[0] is None:
            tails[0] = x.new_zeros((1, x.shape[1], e.conv1.left_pad()))
            tails[1] = x.new_zeros((1, e.conv2.in_channels, e.conv2.left_pad()))
        h, tails[0] = e.conv1.continue_from(x, tails[0])
        h, tails[1] = e.conv2.continue_from(F.gelu(h), tails[1])
        flat = F.gelu(h)[0].transpose(0, 1).contiguous()
        m = flat.shape[0]
        cos, sin = self._rotary(torch.arange(cache.frames, cache.frames + m, device=x.device).float())
        cu = torch.tensor([0, m], dtype=torch.int32, device=x.device)
        for layer, past in zip(self.layers, cache.layers):
            flat = layer(flat, cu, cos, sin, past)
        cache.frames += m
        return self.norm(flat)
