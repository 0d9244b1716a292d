"""Unified understanding + generation model in the style of Bagel: ONE packed decoder carries
text tokens (cross-entropy) and noised VAE-latent patch tokens (flow-matching MSE) in the same
sequence; generation tokens use their own MLP / norm parameters in every layer ("mixture of
transformers"), attention is shared.  Also carries the flow-GRPO pieces used for RL on image
generation: an SDE sampling step that returns its log-probability and the clipped policy / KL
loss.  Reference: src/lmms_engine/models/bagel/bagel.py:199-395 (training forward),
:1046-1360 (``generate_image_learn``, ``_sde_step_with_logprob``),
src/lmms_engine/models/bagel/qwen2_navit.py:243-670 (packed MoT layers)."""
from __future__ import annotations

import math
from dataclasses import dataclass, field, fields
from typing import Any, Dict, List, Optional, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import cross_entropy as ce_ops
from ..ops import attention as attn_ops
from ..ops import gemm as gemm_ops
from ..ops import rope as rope_ops
from .decoder_lm import (IGNORE_INDEX, Attention, DecoderBackbone, DecoderConfig, DecoderLayer, DecoderLM, PackedContext, RMSNorm,
                         SwiGLUMLP, _w, shift_labels_per_document)
from .diffusion import timestep_embedding


ATTN_MODE_NAMES = ("causal", "full", "noise")  # the codes a data pipeline may use instead of the names

LAYER_MODULES = {
    # what the generation tokens own in every layer
    "Qwen2DecoderLayer": (),
    "Qwen2MoEDecoderLayer": ("mlp",),
    "mot_lite": ("mlp", "post_norm"),
    "Qwen2MoTDecoderLayer": ("mlp", "post_norm", "input_norm", "attn", "final_norm"),
}


@dataclass
class BagelConfig(DecoderConfig):
    model_type: str = "bagel"
    latent_channels: int = 16
    latent_patch_size: int = 2
    max_latent_size: int = 64
    timestep_shift: float = 1.0
    ce_weight: float = 1.0
    mse_weight: float = 1.0
    use_mot: bool = True  # without ``layer_module``: True = "mot_lite" (generation tokens own the MLP and its norm)
    layer_module: Optional[str] = None  # a key of LAYER_MODULES; "Qwen2MoTDecoderLayer" is the released model's
    visual_gen: bool = True
    visual_und: bool = False
    vit_config: Optional[Dict[str, Any]] = None
    vit_rope: bool = False
    vit_select_layer: int = -2
    vit_max_num_patch_per_side: int = 70
    connector_act: str = "gelu_pytorch_tanh"
    vae_config: Optional[Dict[str, Any]] = None  # builds the frozen autoencoder inside the model (pixels in, latents inside)
    interpolate_pos: bool = False

    def gen_parts(self):
        name = self.layer_module or ("mot_lite" if self.use_mot else "Qwen2DecoderLayer")
        if name not in LAYER_MODULES:
            raise ValueError(f"unknown layer_module '{name}'; known: {sorted(LAYER_MODULES)}")
        return LAYER_MODULES[name]


def _by_type(x, und, gen, f_und, f_gen):
    """Apply ``f_und`` to the understanding rows and ``f_gen`` to the generation rows of ``x``."""
    parts = []
    if und.numel():
        parts.append((und, f_und(x.index_select(0, und))))
    if gen.numel():
        parts.append((gen, f_gen(x.index_select(0, gen))))
    out = torch.zeros((x.shape[0],) + parts[0][1].shape[1:], dtype=parts[0][1].dtype, device=x.device)
    for idx, val in parts:
        out = out.index_copy(0, idx, val.to(out.dtype))
    return out


class MoTAttention(Attention):
    """Attention whose projections (and QK norms) exist twice; the attention itself is shared, so understanding and
    generation tokens see each other (src/lmms_engine/models/bagel/qwen2_navit.py:396-560)."""

    def __init__(self, cfg: BagelConfig, layer_idx: int):
        super().__init__(cfg, layer_idx)
        H, D = cfg.hidden_size, cfg.head_dim
        self.q_proj_moe_gen = nn.Linear(H, self.n_q * D, bias=cfg.attention_bias)
        self.k_proj_moe_gen = nn.Linear(H, self.n_kv * D, bias=cfg.attention_bias)
        self.v_proj_moe_gen = nn.Linear(H, self.n_kv * D, bias=cfg.attention_bias)
        self.o_proj_moe_gen = nn.Linear(self.n_q * D, H, bias=False)
        if cfg.qk_norm:
            self.q_norm_moe_gen, self.k_norm_moe_gen = RMSNorm(D, cfg.rms_norm_eps), RMSNorm(D, cfg.rms_norm_eps)

    def _qkv(self, x, q, k, v):
        w = torch.cat([q.weight, k.weight, v.weight], 0)
        b = torch.cat([q.bias, k.bias, v.bias], 0) if q.bias is not None else None
        return gemm_ops.linear(x, w, b)

    def forward(self, x, ctx: PackedContext):
        gen = getattr(ctx, "gen_index", None)
        if gen is None:
            return super().forward(x, ctx)
        und, D = ctx.und_index, self.head_dim
        nq, nkv = self.n_q * D, self.n_kv * D
        qkv = _by_type(x, und, gen, lambda t: self._qkv(t, self.q_proj, self.k_proj, self.v_proj),
                       lambda t: self._qkv(t, self.q_proj_moe_gen, self.k_proj_moe_gen, self.v_proj_moe_gen))
        T = qkv.shape[0]
        q, k, v = qkv[:, :nq].reshape(T, self.n_q, D), qkv[:, nq:nq + nkv].reshape(T, self.n_kv, D), qkv[:, nq + nkv:].reshape(T, self.n_kv, D)
        if self.cfg.qk_norm:
            q = _by_type(q, und, gen, lambda t: self.q_norm(t.reshape(-1, D)).view(t.shape), lambda t: self.q_norm_moe_gen(t.reshape(-1, D)).view(t.shape))
            k = _by_type(k, und, gen, lambda t: self.k_norm(t.reshape(-1, D)).view(t.shape), lambda t: self.k_norm_moe_gen(t.reshape(-1, D)).view(t.shape))
        q, k = rope_ops.rope_apply(q.contiguous(), ctx.cos, ctx.sin), rope_ops.rope_apply(k.contiguous(), ctx.cos, ctx.sin)
        o = split_attention(q, k, v.contiguous(), ctx, 1.0 / math.sqrt(D), self.layer_idx).reshape(T, nq)
        return _by_type(o, und, gen, lambda t: gemm_ops.linear(t, self.o_proj.weight, None), lambda t: gemm_ops.linear(t, self.o_proj_moe_gen.weight, None))


def _own_attention_path(ctx) -> bool:
    """Per-split rules, a recorded prefix or a recording pass: all are served by ``split_attention``."""
    return any(getattr(ctx, name, None) is not None for name in ("split_plan", "kv_prefix", "kv_capture"))


def split_attention(q, k, v, ctx: PackedContext, scale: float, layer_idx: int = 0):
    """Attention under the per-split rules when the context carries them, plain packed causal attention otherwise.

    Two hooks serve sampling (the roles of ``NaiveCache`` in src/lmms_engine/models/bagel/modeling_utils.py and of the
    ``forward_cache_update_*`` passes of bagel.py): with ``ctx.kv_capture`` (a list) the rotated keys and the values of
    this layer are recorded; with ``ctx.kv_prefix`` (one ``(k, v)`` per layer) the stream is ONE block that attends
    fully to itself and to that recorded prefix."""
    capture = getattr(ctx, "kv_capture", None)
    if capture is not None:
        capture.append((k.detach(), v.detach()))
    prefix = getattr(ctx, "kv_prefix", None)
    if prefix is not None:
        pk, pv = prefix[layer_idx]
        kk, vv = torch.cat([pk.to(k.dtype), k], 0), torch.cat([pv.to(v.dtype), v], 0)
        cu_q = torch.tensor([0, q.shape[0]], dtype=torch.int32, device=q.device)
        cu_k = torch.tensor([0, kk.shape[0]], dtype=torch.int32, device=q.device)
        # an image block sees itself fully; appended text is causal inside itself (the kernel aligns the mask bottom-right)
        return attn_ops.varlen_attn(q, kk, vv, cu_q, cu_k, causal=bool(getattr(ctx, "kv_prefix_causal", False)), softmax_scale=scale)
    plan = getattr(ctx, "split_plan", None)
    if plan is None:
        return attn_ops.varlen_attn(q, k, v, ctx.cu_seqlens, ctx.cu_seqlens, ctx.max_seqlen, ctx.max_seqlen, causal=True, softmax_scale=scale)
    out = torch.zeros_like(q)
    for q_idx, k_idx, cu_q, cu_k, causal in plan:
        o = attn_ops.varlen_attn(q.index_select(0, q_idx), k.index_select(0, k_idx), v.index_select(0, k_idx), cu_q, cu_k,
                                 causal=causal, softmax_scale=scale)
        out = out.index_copy(0, q_idx, o)
    return out


def build_split_plan(sample_lens: Sequence[int], split_lens: Sequence[int], attn_modes: Sequence[str], device):
    """Turn the per-split attention rules into calls of the packed varlen kernel.

    A sample is a run of splits.  A split sees every earlier split of its sample except "noise" ones, and itself:
    causally ("causal") or fully ("full", "noise"); a "noise" split is seen by nobody else
    (src/lmms_engine/models/bagel/data_utils.py:73-103).  With the kernel's bottom-right aligned causal mask, a split
    becomes one "document" whose queries are its own tokens and whose keys are the visible earlier tokens followed by
    its own; causal and full documents go into two calls.  Keys are gathered per document, so the dense
    ``[T, T]`` mask of the reference is never built."""
    plans = {True: ([], [], [0], [0]), False: ([], [], [0], [0])}
    tok, si = 0, 0
    for n in sample_lens:
        end, visible = tok + n, []
        while tok < end:
            if si >= len(split_lens):
                raise ValueError("split_lens do not cover the samples")
            L, mode = int(split_lens[si]), attn_modes[si]
            if mode not in ("causal", "full", "noise"):
                raise ValueError(f"unknown attention mode '{mode}'")
            own = torch.arange(tok, tok + L)
            qs, ks, cq, ck = plans[mode == "causal"]
            qs.append(own)
            ks.append(torch.cat(visible + [own]) if visible else own)
            cq.append(cq[-1] + L)
            ck.append(ck[-1] + ks[-1].numel())
            if mode != "noise":
                visible.append(own)
            tok, si = tok + L, si + 1
        if tok != end:
            raise ValueError("a split crosses a sample boundary")
    out = []
    for causal, (qs, ks, cq, ck) in plans.items():
        if qs:
            out.append((torch.cat(qs).to(device), torch.cat(ks).to(device), torch.tensor(cq, dtype=torch.int32, device=device),
                        torch.tensor(ck, dtype=torch.int32, device=device), causal))
    return out


class MoTLayer(DecoderLayer):
    """Decoder layer in which generation (latent) tokens own some of the parameters: the MLP ("Qwen2MoEDecoderLayer"),
    also its norm ("mot_lite"), or everything but the attention itself ("Qwen2MoTDecoderLayer")."""

    def __init__(self, cfg: BagelConfig, layer_idx: int):
        super().__init__(cfg, layer_idx)
        parts = cfg.gen_parts()
        self.parts = parts
        if "attn" in parts:
            self.self_attn = MoTAttention(cfg, layer_idx)
        if "mlp" in parts:
            self.mlp_moe_gen = SwiGLUMLP(cfg.hidden_size, cfg.intermediate_size)
        if "post_norm" in parts:
            self.post_attention_layernorm_moe_gen = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps)
        if "input_norm" in parts:
            self.input_layernorm_moe_gen = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps)

    def forward(self, h, residual, ctx: PackedContext):
        gen = getattr(ctx, "gen_index", None)
        if gen is None or not self.parts:
            if not _own_attention_path(ctx):
                return super().forward(h, residual, ctx)
        stream = h if residual is None else h + residual
        und = ctx.und_index if gen is not None else None
        if gen is not None and "input_norm" in self.parts:
            x = _by_type(stream, und, gen, self.input_layernorm, self.input_layernorm_moe_gen)
        else:
            x = self.input_layernorm(stream)
        if isinstance(self.self_attn, MoTAttention) and gen is not None:
            a = self.self_attn(x, ctx)
        else:
            a = self._shared_attention(x, ctx)
        stream = stream + a
        post_g = self.post_attention_layernorm_moe_gen if "post_norm" in self.parts else self.post_attention_layernorm
        mlp_g = self.mlp_moe_gen if "mlp" in self.parts else self.mlp
        if gen is None:
            return self.mlp(self.post_attention_layernorm(stream)), stream
        out = _by_type(stream, und, gen, lambda t: self.mlp(self.post_attention_layernorm(t)), lambda t: mlp_g(post_g(t)))
        return out, stream

    def _shared_attention(self, x, ctx):
        at, D = self.self_attn, self.self_attn.head_dim
        if not _own_attention_path(ctx):
            return at(x, ctx)
        w = torch.cat([_w(at.q_proj.weight), _w(at.k_proj.weight), _w(at.v_proj.weight)], 0)
        b = torch.cat([_w(at.q_proj.bias), _w(at.k_proj.bias), _w(at.v_proj.bias)], 0) if at.q_proj.bias is not None else None
        qkv = gemm_ops.linear(x, w, b)
        T, nq, nkv = qkv.shape[0], at.n_q * D, at.n_kv * D
        q, k, v = qkv[:, :nq].reshape(T, at.n_q, D), qkv[:, nq:nq + nkv].reshape(T, at.n_kv, D), qkv[:, nq + nkv:].reshape(T, at.n_kv, D)
        if at.cfg.qk_norm:
            q, k = at.q_norm(q.reshape(-1, D)).view(q.shape), at.k_norm(k.reshape(-1, D)).view(k.shape)
        q, k = rope_ops.rope_apply(q.contiguous(), ctx.cos, ctx.sin), rope_ops.rope_apply(k.contiguous(), ctx.cos, ctx.sin)
        o = split_attention(q, k, v.contiguous(), ctx, 1.0 / math.sqrt(D), at.layer_idx)
        return gemm_ops.linear(o.reshape(T, nq), _w(at.o_proj.weight), None)


class BagelBackbone(DecoderBackbone):
    layer_cls = MoTLayer

    def __init__(self, cfg: BagelConfig):
        super().__init__(cfg)
        if "final_norm" in cfg.gen_parts():
            self.norm_moe_gen = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps)

    def forward(self, inputs_embeds, ctx: PackedContext):
        gen = getattr(ctx, "gen_index", None)
        if gen is None or not hasattr(self, "norm_moe_gen"):
            return super().forward(inputs_embeds, ctx)
        h, residual = inputs_embeds, None
        for layer in self.layers:
            if self.gradient_checkpointing and self.training:
                h, residual = torch.utils.checkpoint.checkpoint(layer, h, residual, ctx, use_reentrant=False)
            else:
                h, residual = layer(h, residual, ctx)
        return _by_type(h + residual, ctx.und_index, gen, self.norm, self.norm_moe_gen)


class SinCosPositionTable(nn.Module):
    """Frozen 2-D sin-cos table over a ``side x side`` grid, looked up by ``row * side + column``: first half of the
    channels from the column index, second half from the row index (sines then cosines in each)."""

    def __init__(self, side: int, dim: int):
        super().__init__()
        def one(d, pos):
            omega = 1.0 / 10000 ** (torch.arange(d // 2, dtype=torch.float64) / (d / 2.0))
            out = pos.reshape(-1, 1).double() * omega[None]
            return torch.cat([out.sin(), out.cos()], 1)

        rows, cols = torch.meshgrid(torch.arange(side), torch.arange(side), indexing="ij")
        table = torch.cat([one(dim // 2, cols), one(dim // 2, rows)], 1).float()
        self.pos_embed = nn.Parameter(table, requires_grad=False)

    def forward(self, ids):
        return self.pos_embed[ids]


class _TimeEmbedder(nn.Module):
    def __init__(self, hidden: int, freq: int = 256):
        super().__init__()
        self.freq = freq
        self.mlp = nn.Sequential(nn.Linear(freq, hidden), nn.SiLU(), nn.Linear(hidden, hidden))

    def forward(self, t):
        return self.mlp(timestep_embedding(t, self.freq).to(self.mlp[0].weight.dtype))


class _Connector(nn.Module):
    def __init__(self, d_in, d_out, act: str):
        super().__init__()
        self.fc1, self.fc2, self.act = nn.Linear(d_in, d_out), nn.Linear(d_out, d_out), act

    def forward(self, x):
        h = gemm_ops.linear(x, self.fc1.weight, self.fc1.bias)
        h = F.gelu(h, approximate="tanh") if "tanh" in self.act else F.gelu(h)
        return gemm_ops.linear(h, self.fc2.weight, self.fc2.bias)


class BagelContext:
    """What has been said so far, as every layer's rotated keys and values, with the next rotary position."""

    def __init__(self):
        self.layers: Optional[List[Any]] = None
        self.next_pos = 0
        self.length = 0
        self.last_hidden: Optional[torch.Tensor] = None


class TaylorForecaster:
    """Skips decoder passes during sampling by extrapolating the predicted velocity over the step index.

    The first ``first_enhance`` steps are computed; afterwards every ``interval``-th step is, and the steps between are
    forecast from a Taylor expansion whose derivatives (up to ``max_order``) are finite differences of the computed
    steps.  This is the schedule and the expansion of the reference's TaylorSeer option
    (src/lmms_engine/models/bagel/cache_utils.py:12-128, qwen2_navit.py:839-908), applied to the velocity of the latent
    tokens - the quantity the sampler consumes - instead of to every layer's output, of which only the last one reaches
    the result; one forecaster serves one guidance branch."""

    def __init__(self, interval: int = 3, max_order: int = 6, first_enhance: int = 5):
        self.interval, self.max_order, self.first_enhance = max(int(interval), 1), int(max_order), int(first_enhance)
        self.factors: List[torch.Tensor] = []
        self.computed: List[int] = []
        self.counter = 0

    def wants_model(self, step: int) -> bool:
        """Whether ``step`` must run the model; otherwise ``forecast`` serves it.  Call once per step, in order."""
        if step < self.first_enhance or self.counter == self.interval - 1 or not self.factors:
            self.counter = 0
            return True
        self.counter += 1
        return False

    def update(self, step: int, value: torch.Tensor) -> None:
        new = [value]
        if self.computed and step > self.first_enhance - 2:
            distance = step - self.computed[-1]
            for i in range(min(self.max_order, len(self.factors))):
                new.append((new[i] - self.factors[i]) / distance)
        self.factors = new
        self.computed.append(step)

    def forecast(self, step: int) -> torch.Tensor:
        x = step - self.computed[-1]
        return sum(f * (x ** i / math.factorial(i)) for i, f in enumerate(self.factors))


class Bagel(DecoderLM):
    supports_kv_cache = False
    config_class = BagelConfig
    backbone_cls = BagelBackbone
    _no_split_modules = ["MoTLayer"]

    def __init__(self, cfg: BagelConfig):
        super().__init__(cfg)
        pd = cfg.latent_channels * cfg.latent_patch_size ** 2
        if cfg.visual_gen:
            self.vae2llm = nn.Linear(pd, cfg.hidden_size)
            self.llm2vae = nn.Linear(cfg.hidden_size, pd)
            self.time_embedder = _TimeEmbedder(cfg.hidden_size)
            self.latent_pos_embed = SinCosPositionTable(cfg.max_latent_size, cfg.hidden_size)
        if cfg.visual_und:
            from .bagel_parts import SiglipNavit
            from .llava_ov import SiglipConfig

            vc = SiglipConfig.from_dict(cfg.vit_config or {})
            self.vit_model = SiglipNavit(vc, rope=cfg.vit_rope, select_layer=cfg.vit_select_layer)
            self.connector = _Connector(vc.hidden_size, cfg.hidden_size, cfg.connector_act)
            self.vit_pos_embed = SinCosPositionTable(cfg.vit_max_num_patch_per_side, cfg.hidden_size)
        self.vae_model = None
        if cfg.vae_config is not None:
            from .bagel_parts import AutoEncoderParams, BagelAutoEncoder

            params = AutoEncoderParams.from_dict(dict(cfg.vae_config, z_channels=cfg.latent_channels))
            self.vae_model = BagelAutoEncoder(params).requires_grad_(False).eval()

    def train(self, mode: bool = True):
        super().train(mode)
        if self.vae_model is not None:
            self.vae_model.eval()
        return self

    # ---- inputs -------------------------------------------------------------------------------------------
    @torch.no_grad()
    def latents_from_images(self, images, latent_shapes):
        """Pixels ``[n, 3, H, W]`` (padded to a common size, in ``[-1, 1]``) -> packed latent patches ``[G, C*p*p]`` in
        row-major patch order with (pixel row, pixel column, channel) inside a patch, cropped to each image's ``(h, w)``
        patch grid."""
        if self.vae_model is None:
            raise ValueError("images were given but the model has no autoencoder (set vae_config or feed latent_tokens)")
        p, C = self.config.latent_patch_size, self.config.latent_channels
        z = self.vae_model.encode(images.to(next(self.vae_model.parameters()).dtype))
        out = []
        for lat, (h, w) in zip(z, latent_shapes):
            h, w = int(h), int(w)
            out.append(lat[:, : h * p, : w * p].reshape(C, h, p, w, p).permute(1, 3, 2, 4, 0).reshape(h * w, p * p * C))
        return torch.cat(out, 0)

    def embed_stream(self, ids, latent_tokens=None, latent_index=None, latent_pos=None, timesteps=None, vit_tokens=None,
                     vit_index=None, vit_position_ids=None, vit_seqlens=None, noise=None):
        """Token embeddings with the image rows written in.  Returns ``(emb, noise, target, t)``."""
        cfg = self.config
        emb = self.model.embed_tokens(ids)
        if vit_tokens is not None:
            if not cfg.visual_und:
                raise ValueError("understanding image tokens were given to a model built with visual_und = False")
            cu = F.pad(torch.cumsum(vit_seqlens.to(torch.int32), 0, dtype=torch.int32), (1, 0))
            v = self.vit_model(vit_tokens, vit_position_ids, cu)
            v = self.connector(v) + self.vit_pos_embed(vit_position_ids).to(v.dtype)
            emb = emb.index_copy(0, vit_index, v.to(emb.dtype))
        target = t = None
        if latent_tokens is not None and latent_tokens.shape[0]:
            clean = latent_tokens.float()
            t = timesteps.float()
            t = cfg.timestep_shift * t / (1 + (cfg.timestep_shift - 1) * t)
            noise = torch.randn_like(clean) if noise is None else noise.float()
            x_t = (1 - t[:, None]) * clean + t[:, None] * noise
            target = noise - clean
            g = self.vae2llm(x_t.to(emb.dtype)) + self.time_embedder(t).to(emb.dtype) + self.latent_pos_embed(latent_pos).to(emb.dtype)
            emb = emb.index_copy(0, latent_index, g)
        return emb, noise, target, t

    def run_decoder(self, emb, pos, cu, gen_index, split_lens=None, attn_modes=None, kv_capture=None, kv_prefix=None,
                    prefix_causal: bool = False):
        cos, sin = self.model.rope_tables(pos)
        ctx = PackedContext(cu, int(pos.shape[-1]), cos, sin, True)
        if kv_capture is not None:
            ctx.kv_capture = kv_capture
        if kv_prefix is not None:
            ctx.kv_prefix, ctx.kv_prefix_causal = kv_prefix, prefix_causal
        T = emb.shape[0]
        if gen_index is not None and gen_index.numel() and self.config.gen_parts():
            mask = torch.zeros(T, dtype=torch.bool, device=emb.device)
            mask[gen_index] = True
            ctx.gen_index = gen_index
            ctx.und_index = torch.nonzero(~mask, as_tuple=False).flatten()
        if split_lens is not None:
            lens = (cu[1:] - cu[:-1]).tolist()
            modes = attn_modes.tolist() if torch.is_tensor(attn_modes) else list(attn_modes)
            modes = [ATTN_MODE_NAMES[m] if isinstance(m, int) else m for m in modes]
            sl = split_lens.tolist() if torch.is_tensor(split_lens) else list(split_lens)
            ctx.split_plan = build_split_plan(lens, sl, modes, emb.device)
        return self.model(emb, ctx)

    def forward(self, input_ids=None, labels=None, cu_seqlens=None, position_ids=None, latent_tokens=None,
                latent_index=None, latent_pos=None, timesteps=None, latent_loss_mask=None, vit_tokens=None, vit_index=None,
                vit_position_ids=None, vit_seqlens=None, images=None, latent_shapes=None, split_lens=None, attn_modes=None,
                noise=None, **kw) -> Dict[str, Any]:
        """Packed stream of length T.  ``latent_tokens [G, C*p*p]`` are clean autoencoder patches (or ``images`` +
        ``latent_shapes`` to encode them here) that sit at stream positions ``latent_index [G]`` (their ``input_ids``
        entries are ignored); ``timesteps [G]`` in (0, 1) give each patch's noise level (0 = a clean condition image,
        which carries no loss).  ``vit_*`` place packed SigLIP tokens of understanding images.  ``split_lens`` /
        ``attn_modes`` give every sample's attention rules (causal text, full images, invisible noised images);
        without them the stream is plainly causal."""
        cfg = self.config
        ids, labels, pos, cu, _ = self.prepare_packed(input_ids, None, labels, position_ids, cu_seqlens)
        if latent_tokens is None and images is not None:
            latent_tokens = self.latents_from_images(images, latent_shapes)
        emb, noise, target, t = self.embed_stream(ids, latent_tokens, latent_index, latent_pos, timesteps, vit_tokens, vit_index,
                                                  vit_position_ids, vit_seqlens, noise)
        G = 0 if target is None else target.shape[0]
        hidden = self.run_decoder(emb, pos, cu, latent_index if G else None, split_lens, attn_modes)
        out: Dict[str, Any] = {}
        ce = mse = None
        if labels is not None:
            shifted = shift_labels_per_document(labels, cu)
            ce = ce_ops.fused_linear_cross_entropy(hidden, _w(self.lm_head.weight), shifted, "mean")
        if G:
            pred = self.llm2vae(hidden.index_select(0, latent_index)).float()
            err = ((pred - target) ** 2).mean(-1)
            keep = (t > 0).to(err.dtype)  # clean condition images carry no loss
            if latent_loss_mask is not None:
                keep = keep * latent_loss_mask.to(err.dtype)
            mse = (err * keep).sum() / keep.sum().clamp(min=1.0)
            out["velocity"] = pred
        loss = 0.0
        if ce is not None:
            loss = loss + cfg.ce_weight * ce
        if mse is not None:
            loss = loss + cfg.mse_weight * mse
        out.update(loss=loss, ce=ce.detach() if ce is not None else None, mse=mse.detach() if mse is not None else None)
        return out

    def convert_hf_state_dict(self, sd: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        """Released checkpoints nest the decoder under ``language_model.`` and hold the patch convolution of the SigLIP
        tower either way; everything else has this module's names."""
        out = {}
        for k, v in sd.items():
            if k.startswith("language_model."):
                k = k[len("language_model."):]
            if k.endswith("vit_model.vision_model.embeddings.patch_embedding.weight") and v.dim() == 4:
                v = v.permute(0, 2, 3, 1).reshape(v.shape[0], -1)
            out[k] = v
        return out

    # ---- image generation and its policy-gradient pass ----------------------------------------------------
    def image_stream(self, prompt_ids: torch.Tensor, hw, boi_id: int, eoi_id: int):
        """Packed inputs of "prompt, then one image to generate": the prompt is causal text, the image block
        (begin marker, ``h*w`` latent tokens, end marker) attends fully to itself and to the prompt and sits at ONE rotary
        position, like every image of the training streams."""
        h, w = int(hw[0]), int(hw[1])
        dev, n, G = prompt_ids.device, prompt_ids.numel(), h * w
        ids = torch.cat([prompt_ids, torch.tensor([boi_id] + [0] * G + [eoi_id], device=dev, dtype=prompt_ids.dtype)])
        pos = torch.cat([torch.arange(n, device=dev), torch.full((G + 2,), n, device=dev)])
        side = self.config.max_latent_size
        lat_pos = (torch.arange(h, device=dev)[:, None] * side + torch.arange(w, device=dev)[None]).flatten()
        return dict(ids=ids, pos=pos, cu=torch.tensor([0, n + G + 2], dtype=torch.int32, device=dev), latent_index=torch.arange(n + 1, n + 1 + G, device=dev),
                    latent_pos=lat_pos, split_lens=[n, G + 2] if n else [G + 2], attn_modes=["causal", "full"] if n else ["full"])

    # ---- a conversation kept as keys / values: text, understood images and condition images appended turn by turn ----
    @torch.no_grad()
    def extend_context(self, context: Optional["BagelContext"], emb, pos, gen_index=None, causal: bool = True):
        """Append one chunk (already embedded) to ``context``: it attends to everything appended before and to itself
        (``causal``: text; otherwise fully: an image block).  Returns the chunk's hidden states.  The role of the
        reference's ``forward_cache_update_text / _vit / _vae`` (src/lmms_engine/models/bagel/bagel.py:396-700)."""
        context = context if context is not None else BagelContext()
        T = emb.shape[0]
        cu = torch.tensor([0, T], dtype=torch.int32, device=emb.device)
        captured: List[Any] = []
        if context.layers is None:
            hidden = self.run_decoder(emb, pos, cu, gen_index, [T], ["causal" if causal else "full"], kv_capture=captured)
            context.layers = captured
        else:
            hidden = self.run_decoder(emb, pos, cu, gen_index, kv_capture=captured, kv_prefix=context.layers, prefix_causal=causal)
            context.layers = [(torch.cat([pk, k], 0), torch.cat([pv, v], 0)) for (pk, pv), (k, v) in zip(context.layers, captured)]
        if len(context.layers) != len(self.model.layers):
            raise RuntimeError(f"{len(context.layers)} layers recorded their keys, the decoder has {len(self.model.layers)}")
        context.length += T
        context.last_hidden = hidden
        return context

    @torch.no_grad()
    def add_text(self, context, ids: torch.Tensor):
        context = context if context is not None else BagelContext()
        n = ids.numel()
        pos = torch.arange(context.next_pos, context.next_pos + n, device=ids.device)
        context = self.extend_context(context, self.model.embed_tokens(ids.reshape(-1)), pos, None, causal=True)
        context.next_pos += n
        return context

    @torch.no_grad()
    def add_image(self, context, boi_id: int, eoi_id: int, latent_tokens=None, latent_pos=None, vit_tokens=None, vit_position_ids=None):
        """Append one image block ``begin marker, image rows, end marker`` at ONE rotary position: ``vit_tokens`` (an image to
        understand: packed SigLIP patches of that image) or ``latent_tokens`` (a clean condition image: autoencoder patches at
        noise level 0, handled by the generation parameters)."""
        context = context if context is not None else BagelContext()
        dev = (latent_tokens if latent_tokens is not None else vit_tokens).device
        rows = (latent_tokens if latent_tokens is not None else vit_tokens).shape[0]
        ids = torch.tensor([boi_id] + [0] * rows + [eoi_id], device=dev)
        inner = torch.arange(1, rows + 1, device=dev)
        if latent_tokens is not None:
            emb, _, _, _ = self.embed_stream(ids, latent_tokens, inner, latent_pos, torch.zeros(rows, device=dev), noise=torch.zeros_like(latent_tokens.float()))
            gen = inner
        else:
            emb, _, _, _ = self.embed_stream(ids, vit_tokens=vit_tokens, vit_index=inner, vit_position_ids=vit_position_ids,
                                             vit_seqlens=torch.tensor([rows], device=dev))
            gen = None
        pos = torch.full((rows + 2,), context.next_pos, device=dev)
        context = self.extend_context(context, emb, pos, gen, causal=False)
        context.next_pos += 1
        return context

    @torch.no_grad()
    def cache_prompt(self, stream: Dict[str, Any]) -> Dict[str, Any]:
        """Run the prompt of ``stream`` once and keep every layer's rotated keys and values, so that the sampling steps
        only run the image block against them.  Exact: the prompt is causal text in front of the block, so nothing in
        it depends on the block.  Returns ``stream`` with ``prefix`` (one ``(k, v)`` per layer) and ``block`` (the
        stream reduced to the image block); a stream without a prompt is returned unchanged."""
        n = int(stream["latent_index"][0]) - 1  # tokens in front of the begin-of-image marker
        if n <= 0 or "prefix" in stream:
            return stream
        captured: List[Any] = []
        emb = self.model.embed_tokens(stream["ids"][:n])
        cu = torch.tensor([0, n], dtype=torch.int32, device=emb.device)
        self.run_decoder(emb, stream["pos"][:n], cu, None, [n], ["causal"], kv_capture=captured)
        if len(captured) != len(self.model.layers):
            raise RuntimeError(f"{len(captured)} layers recorded their keys, the decoder has {len(self.model.layers)}")
        block = dict(ids=stream["ids"][n:], pos=stream["pos"][n:], latent_index=stream["latent_index"] - n, latent_pos=stream["latent_pos"],
                     cu=torch.tensor([0, stream["ids"].numel() - n], dtype=torch.int32, device=emb.device))
        return dict(stream, prefix=captured, block=block)

    def _block_after(self, context: "BagelContext", hw, boi_id: int, eoi_id: int, dev) -> Dict[str, Any]:
        """The image block that follows ``context``, in the form ``flow_velocity`` runs against recorded keys / values."""
        bare = self.image_stream(torch.zeros(0, dtype=torch.long, device=dev), hw, boi_id, eoi_id)
        block = dict(ids=bare["ids"], pos=bare["pos"] + context.next_pos, latent_index=bare["latent_index"], latent_pos=bare["latent_pos"], cu=bare["cu"])
        return dict(bare, prefix=context.layers, block=block)

    def flow_velocity(self, stream: Dict[str, Any], x_t: torch.Tensor, t: float, cached: bool = False) -> torch.Tensor:
        """Velocity prediction ``[G, C*p*p]`` for the noised latent patches ``x_t`` of ``stream`` at time ``t`` in (0, 1].
        ``cached``: use the prompt keys / values recorded by ``cache_prompt`` (sampling only: they carry no gradient)."""
        prefix = stream.get("prefix") if cached else None
        part = stream["block"] if prefix is not None else stream
        emb = self.model.embed_tokens(part["ids"])
        tt = torch.full((x_t.shape[0],), float(t), device=x_t.device)
        g = self.vae2llm(x_t.to(emb.dtype)) + self.time_embedder(tt).to(emb.dtype) + self.latent_pos_embed(part["latent_pos"]).to(emb.dtype)
        emb = emb.index_copy(0, part["latent_index"], g)
        if prefix is not None:
            hidden = self.run_decoder(emb, part["pos"], part["cu"], part["latent_index"], kv_prefix=prefix)
        else:
            hidden = self.run_decoder(emb, part["pos"], part["cu"], part["latent_index"], part["split_lens"], part["attn_modes"])
        return self.llm2vae(hidden.index_select(0, part["latent_index"])).float()

    def guided_velocity(self, stream, x_t, t, uncond_stream=None, cfg_text_scale: float = 1.0, cfg_renorm_min: float = 0.0,
                        cfg_renorm_type: str = "global", cached: bool = False, forecast=None):
        """Classifier-free guidance on the text condition with the guided field rescaled down to the conditional one's
        norm (over everything: "global"; per token: "channel").  ``forecast = (step, forecaster of the conditional
        branch, forecaster of the unconditional branch)`` lets the forecasters serve the steps they can."""

        def branch(st, fc):
            if fc is None:
                return self.flow_velocity(st, x_t, t, cached)
            if fc.wants_model(forecast[0]):
                v = self.flow_velocity(st, x_t, t, cached)
                fc.update(forecast[0], v)
                return v
            return fc.forecast(forecast[0])

        v = branch(stream, forecast[1] if forecast else None)
        if uncond_stream is None or cfg_text_scale <= 1.0:
            return v
        v_un = branch(uncond_stream, forecast[2] if forecast else None)
        v_g = v_un + cfg_text_scale * (v - v_un)
        if cfg_renorm_type == "global":
            scale = (v.norm() / (v_g.norm() + 1e-8)).clamp(min=cfg_renorm_min, max=1.0)
        elif cfg_renorm_type == "channel":
            scale = (v.norm(dim=-1, keepdim=True) / (v_g.norm(dim=-1, keepdim=True) + 1e-8)).clamp(min=cfg_renorm_min, max=1.0)
        else:
            raise ValueError(f"unknown cfg_renorm_type '{cfg_renorm_type}' (global | channel)")
        return v_g * scale

    def flow_schedule(self, num_timesteps: int, device, timestep_shift: Optional[float] = None):
        s = self.config.timestep_shift if timestep_shift is None else timestep_shift
        t = torch.linspace(1, 0, num_timesteps, device=device)
        return s * t / (1 + (s - 1) * t)

    @torch.no_grad()
    def generate_image(self, prompt_ids, hw, boi_id: int, eoi_id: int, num_timesteps: int = 24, timestep_shift: Optional[float] = None,
                       noise_level: float = 0.7, sde_window=None, uncond_ids=None, cfg_text_scale: float = 1.0, cfg_interval=(0.0, 1.0),
                       cfg_renorm_min: float = 0.0, cfg_renorm_type: str = "global", generator=None, use_cache: bool = True,
                       taylor: Optional[Dict[str, int]] = None, context: Optional["BagelContext"] = None,
                       uncond_context: Optional["BagelContext"] = None) -> Dict[str, Any]:
        """Sample one image's latent patches from noise.  Steps inside ``sde_window = (first, count)`` (default: all) are
        stochastic and recorded - the state before the step, the state after it, its time and its log-probability - for
        the policy-gradient pass; the other steps are plain Euler steps of the flow.  ``use_cache``: run the prompt once
        and every step on the image block only (same result; the recorded streams stay complete for the learning pass).
        ``taylor`` (``{"interval", "max_order", "first_enhance"}``, any subset): forecast the velocity of the steps between
        computed ones (``TaylorForecaster``; approximate, meant for previews and evaluation, not for recorded rollouts)."""
        if context is not None:
            # the image follows a conversation held as keys / values (``add_text`` / ``add_image``): the recorded streams
            # are blocks only, so such a rollout cannot feed ``grpo_learn``
            dev = context.layers[0][0].device
            stream = self._block_after(context, hw, boi_id, eoi_id, dev)
            un = self._block_after(uncond_context, hw, boi_id, eoi_id, dev) if uncond_context is not None else None
            use_cache = True
        else:
            dev = prompt_ids.device
            stream = self.image_stream(prompt_ids, hw, boi_id, eoi_id)
            un = self.image_stream(uncond_ids, hw, boi_id, eoi_id) if uncond_ids is not None else None
            if use_cache:
                stream = self.cache_prompt(stream)
                un = self.cache_prompt(un) if un is not None else None
        ts = self.flow_schedule(num_timesteps, dev, timestep_shift)
        pd = self.config.latent_channels * self.config.latent_patch_size ** 2
        x = torch.randn((int(hw[0]) * int(hw[1]), pd), device=dev, generator=generator)
        first, count = sde_window if sde_window is not None else (0, num_timesteps - 1)
        rec: Dict[str, List] = {"latents": [], "prev_latents": [], "timesteps": [], "next_timesteps": [], "log_probs": []}
        seers = (TaylorForecaster(**taylor), TaylorForecaster(**taylor)) if taylor is not None else None
        for i in range(num_timesteps - 1):
            t, t_next = float(ts[i]), float(ts[i + 1])
            scale = cfg_text_scale if cfg_interval[0] < t <= cfg_interval[1] else 1.0
            v = self.guided_velocity(stream, x, t, un, scale, cfg_renorm_min, cfg_renorm_type, cached=use_cache,
                                     forecast=(i,) + seers if seers else None)
            if first <= i < first + count and noise_level > 0:
                nxt, logp, _, _ = self.sde_step_with_logprob(v[None], x[None], torch.tensor([t], device=dev), t_next - t, noise_level,
                                                             generator=generator, sigma_max=float(ts[1]))
                rec["latents"].append(x)
                rec["prev_latents"].append(nxt[0])
                rec["timesteps"].append(t)
                rec["next_timesteps"].append(t_next)
                rec["log_probs"].append(logp[0])
                x = nxt[0]
            else:
                x = x + v * (t_next - t)
        rec["image_latent"] = x
        plain = lambda st: None if st is None else {k: v for k, v in st.items() if k not in ("prefix", "block")}  # noqa: E731
        rec["stream"], rec["uncond_stream"] = plain(stream), plain(un)
        return rec

    def unpatchify_latent(self, tokens: torch.Tensor, hw) -> torch.Tensor:
        """Packed latent patches ``[h*w, p*p*C]`` -> ``[C, h*p, w*p]`` (decode with the autoencoder for pixels)."""
        p, C = self.config.latent_patch_size, self.config.latent_channels
        h, w = int(hw[0]), int(hw[1])
        return tokens.view(h, w, p, p, C).permute(4, 0, 2, 1, 3).reshape(C, h * p, w * p)

    def grpo_learn(self, rollout: Dict[str, Any], advantage, clip_range=(1e-4, 1e-4), beta: float = 0.0, ref_model: Optional["Bagel"] = None,
                   noise_level: float = 0.7, cfg_text_scale: float = 1.0, cfg_renorm_min: float = 0.0, cfg_renorm_type: str = "global",
                   adv_clip_max: float = 5.0, step_callback=None) -> Dict[str, torch.Tensor]:
        """Policy-gradient pass over a recorded rollout: for every recorded step the current policy's log-probability of
        the step that was taken, the clipped-ratio loss against the log-probability at sampling time, and (``beta > 0``)
        the closed-form Gaussian KL to ``ref_model``'s step mean.  ``step_callback(loss)`` runs after every step (backward,
        optimizer step); without it the step losses are averaged and returned for one backward."""
        adv = torch.as_tensor(advantage, device=rollout["latents"][0].device, dtype=torch.float32).clamp(-adv_clip_max, adv_clip_max)
        lo, hi = (clip_range, clip_range) if isinstance(clip_range, float) else clip_range
        stats = {"policy_loss": [], "kl_loss": [], "loss": [], "clipfrac": []}
        ts = sorted({*rollout["timesteps"], *rollout["next_timesteps"]}, reverse=True)
        sigma_max = ts[1] if len(ts) > 1 and ts[0] >= 1.0 else None
        for x, nxt, t, t_next, old in zip(rollout["latents"], rollout["prev_latents"], rollout["timesteps"], rollout["next_timesteps"],
                                          rollout["log_probs"]):
            v = self.guided_velocity(rollout["stream"], x, t, rollout.get("uncond_stream"), cfg_text_scale, cfg_renorm_min, cfg_renorm_type)
            tt = torch.tensor([t], device=x.device)
            _, logp, mean, sd = self.sde_step_with_logprob(v[None], x[None], tt, t_next - t, noise_level, prev_sample=nxt[None], sigma_max=sigma_max)
            ratio = torch.exp(logp - old.detach())
            policy = torch.maximum(-adv * ratio, -adv * torch.clamp(ratio, 1 - lo, 1 + hi)).mean()
            loss, kl = policy, policy.new_zeros(())
            if beta > 0 and ref_model is not None:
                with torch.no_grad():
                    v_ref = ref_model.guided_velocity(rollout["stream"], x, t, rollout.get("uncond_stream"), cfg_text_scale, cfg_renorm_min,
                                                      cfg_renorm_type)
                    _, _, mean_ref, _ = self.sde_step_with_logprob(v_ref[None], x[None], tt, t_next - t, noise_level, prev_sample=nxt[None],
                                                                   sigma_max=sigma_max)
                kl = (((mean - mean_ref) ** 2).mean() / (2 * sd.mean() ** 2))
                loss = policy + beta * kl
            stats["policy_loss"].append(policy.detach())
            stats["kl_loss"].append(kl.detach())
            stats["clipfrac"].append(((ratio - 1 > hi) | (1 - ratio > lo)).float().mean().detach())
            if step_callback is not None:
                step_callback(loss)
                stats["loss"].append(loss.detach())
            else:
                stats["loss"].append(loss)
        return {k: torch.stack(v).mean() for k, v in stats.items()}

    # ---- flow-GRPO -----------------------------------------------------------------------------
    @staticmethod
    def sde_step_with_logprob(v, x, t, dt, noise_level: float = 0.7, prev_sample=None, generator=None, sigma_max=None):
        """One reverse-time SDE step of the rectified flow (t: 1 = noise -> 0 = data, ``dt < 0``) together with the Gaussian
        log-probability of the sample it produced, averaged over dimensions.  At ``t = 1`` the noise scale
        ``sqrt(t / (1 - t))`` is evaluated with ``sigma_max`` (the schedule's second time) in the denominator."""
        v, x = v.float(), x.float()
        t = t.float().view(-1, *([1] * (x.dim() - 1)))
        cap = torch.full_like(t, 1 - 1e-3 if sigma_max is None else float(sigma_max))
        std = noise_level * torch.sqrt(t / (1 - torch.where(t >= 1, cap, t)).clamp(min=1e-3))
        mean = x * (1 + std ** 2 / (2 * t) * dt) + v * (1 + std ** 2 * (1 - t) / (2 * t)) * dt
        sd = std * math.sqrt(abs(dt))
        if prev_sample is None:
            prev_sample = mean + sd * torch.randn(x.shape, device=x.device, generator=generator)
        var = sd ** 2 + 1e-8
        logp = -((prev_sample.detach().float() - mean) ** 2) / (2 * var) - 0.5 * torch.log(var) - 0.5 * math.log(2 * math.pi)
        return prev_sample, logp.mean(dim=tuple(range(1, x.dim()))), mean, sd

    @staticmethod
    def grpo_loss(logp, old_logp, advantages, clip_range: float = 1e-4, kl_mean=None, ref_mean=None, sd=None, beta: float = 0.0):
        """Clipped-ratio policy loss (+ closed-form Gaussian KL to the reference policy's step mean)."""
        ratio = torch.exp(logp - old_logp)
        unclipped = -advantages * ratio
        clipped = -advantages * torch.clamp(ratio, 1 - clip_range, 1 + clip_range)
        loss = torch.maximum(unclipped, clipped).mean()
        if beta > 0 and kl_mean is not None:
            kl = ((kl_mean - ref_mean) ** 2).mean(dim=tuple(range(1, kl_mean.dim())), keepdim=True) / (2 * sd ** 2)
            loss = loss + beta * kl.mean()
        return loss


def apply_nsa_to_bagel(model: "Bagel", block_size: int = 64, compress_type: str = "weightedpool", kernel_size: int = 32,
                       kernel_stride: int = 16, topk: int = 16, init_blocks: int = 1, local_blocks: int = 2,
                       window_size: int = 512, **_):
    """Turn every attention layer of a built model into native sparse attention: adds the gate projection
    (three gates per query head), the pooling parameters of the key and value compression and the
    intra-window position term, and records the settings on the config (reference:
    src/lmms_engine/models/bagel/monkey_patch.py:160-253)."""
    from ..ops import nsa as nsa_ops

    params = nsa_ops.NSAParams(block_size, compress_type, kernel_size, kernel_stride, topk, init_blocks, local_blocks, window_size)
    cfg = model.config
    for layer in model.model.layers:
        attn = layer.self_attn
        ref = attn.q_proj.weight
        attn.g_proj = nn.Linear(cfg.hidden_size, attn.n_q * 3, bias=False).to(device=ref.device, dtype=ref.dtype)
        for name in ("compress_key", "compress_value"):
            w = nsa_ops.compress_weight(compress_type, attn.n_kv, attn.head_dim, kernel_size)
            if w is None:
                setattr(attn, name, None)
            else:
                attn.register_parameter(name, nn.Parameter(w.to(device=ref.device, dtype=ref.dtype)))
        attn.register_parameter("intra_block_pe", nn.Parameter(torch.zeros(attn.n_kv, kernel_size, attn.head_dim, device=ref.device, dtype=ref.dtype)))
        attn.nsa = params
    cfg.extra["nsa_config"] = {k: getattr(params, k) for k in params.__dataclass_fields__}
    return model


from .monkey_patch import MONKEY_PATCHER  # noqa: E402

MONKEY_PATCHER.register("bagel", "nsa")(apply_nsa_to_bagel)
