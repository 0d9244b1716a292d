"""Qwen3.5 hybrid decoder: three Gated-DeltaNet (linear attention) layers for every gated softmax-attention layer,
zero-centred RMSNorm, partial rotary embedding (``model_type: qwen3_5_text`` / ``qwen3_5``, text stream).
The reference patches the ``transformers`` classes and delegates the recurrence to the ``fla`` Triton kernels
(src/lmms_engine/models/qwen3_5/qwen3_5_ops.py:138-298 linear attention, :445-529 gated attention).

Gated delta rule per head (state ``S [d_k, d_v]``, decay ``exp(g_t) <= 1``, write strength ``beta_t``):

    S_t = exp(g_t) S_{t-1} + beta_t k_t (v_t - (exp(g_t) S_{t-1})^T k_t)^T,    o_t = S_t^T q_t / sqrt(d_k)

It is evaluated chunk-wise (64 tokens): inside a chunk through the inverse of a unit lower-triangular matrix,
between chunks through the carried state.  All documents of a packed batch are padded to whole chunks and
processed together (``ops/gdn.py``): the in-chunk algebra as batched fp32 ops, the chunk-to-chunk recurrence in one
CUDA kernel per direction with the state reset at every document start, so neither the short causal convolution nor
the state ever crosses a document boundary.  Projections, norms, the gated attention layers and the loss use the
engine's kernels.  Under Ulysses sequence parallelism the heads of both layer kinds are exchanged around the
sequence-wide parts (convolution + rule, attention).  Full-attention heads wider than 128
(the released models use 256) fall back to the reference attention path.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from ..ops import attention as attn_ops
from ..ops import gemm as gemm_ops
from ..ops import gdn as gdn_ops
from ..ops import norm as norm_ops
from ..ops import rope as rope_ops
from ..parallel.sequence_parallel import ulysses as sp
from .decoder_lm import DecoderBackbone, DecoderConfig, DecoderLM, PackedContext, SwiGLUMLP, _w


@dataclass
class Qwen35Config(DecoderConfig):
    model_type: str = "qwen3_5_text"
    partial_rotary_factor: float = 0.25
    linear_conv_kernel_dim: int = 4
    linear_key_head_dim: int = 128
    linear_value_head_dim: int = 128
    linear_num_key_heads: int = 16
    linear_num_value_heads: int = 32
    linear_attn_cp: str = "auto"  # under sequence parallelism: heads | state | auto (see GatedDeltaNet.cp_mode)
    layer_types: Optional[List[str]] = None
    full_attention_interval: int = 4

    def __post_init__(self):
        super().__post_init__()
        if self.layer_types is None:
            k = self.full_attention_interval
            self.layer_types = ["full_attention" if (i + 1) % k == 0 else "linear_attention" for i in range(self.num_hidden_layers)]

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "Qwen35Config":
        d = dict(d.get("text_config") or d)
        rope = d.get("rope_parameters") or d.get("rope_scaling") or {}
        if "partial_rotary_factor" in rope:
            d["partial_rotary_factor"] = rope["partial_rotary_factor"]  # the rope dict is what the hub model reads
        d["model_type"] = d.get("model_type", "qwen3_5_text")
        return super().from_dict(d)


class ZRMSNorm(nn.Module):
    """RMSNorm whose scale is stored as an offset from one (weights initialised to zero)."""

    def __init__(self, dim: int, eps: float = 1e-6):
        super().__init__()
        self.weight = nn.Parameter(torch.zeros(dim))
        self.eps = eps

    def forward(self, x, residual=None):
        return norm_ops.rmsnorm(x, self.weight, self.eps, 1.0, residual)


# ------------------------------------------------------------------------------- gated delta rule
def _l2norm(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    return x * torch.rsqrt((x * x).sum(-1, keepdim=True) + eps)


def chunk_gated_delta_rule(q, k, v, g, beta, chunk: int = 64):
    """``q, k [T, H, dk]``, ``v [T, H, dv]``, ``g, beta [T, H]`` of ONE document -> ``o [T, H, dv]`` (fp32 math)."""
    dt = q.dtype
    q, k = _l2norm(q.float()), _l2norm(k.float())
    q, k, v = (x.transpose(0, 1) for x in (q, k, v.float()))  # [H, T, d]
    g, beta = g.float().transpose(0, 1), beta.float().transpose(0, 1)  # [H, T]
    H, T, dk = k.shape
    dv = v.shape[-1]
    pad = (-T) % chunk
    if pad:
        q, k, v = (F.pad(x, (0, 0, 0, pad)) for x in (q, k, v))
        g, beta = F.pad(g, (0, pad)), F.pad(beta, (0, pad))
    n = (T + pad) // chunk
    q = q * dk ** -0.5
    vb, kb = v * beta[..., None], k * beta[..., None]
    q, k, v, kb, vb = (x.reshape(H, n, chunk, x.shape[-1]) for x in (q, k, v, kb, vb))
    g = g.reshape(H, n, chunk).cumsum(-1)
    decay = (g[..., :, None] - g[..., None, :]).tril().exp().tril()
    # (I + strictly-lower(kb k^T * decay))^-1 by forward substitution on the unit lower-triangular system
    a = (kb @ k.transpose(-1, -2)) * decay
    a = a.masked_fill(torch.triu(torch.ones(chunk, chunk, dtype=torch.bool, device=q.device)), 0)
    eye = torch.eye(chunk, dtype=a.dtype, device=a.device)
    inv = torch.linalg.solve_triangular(eye + a, eye.expand_as(a).contiguous(), upper=False)
    u = inv @ vb                                   # values after the in-chunk corrections
    w = inv @ (kb * g.exp()[..., None])            # what the carried state contributes to them
    state = q.new_zeros((H, dk, dv))
    out = torch.empty_like(u)
    strict = torch.triu(torch.ones(chunk, chunk, dtype=torch.bool, device=q.device), diagonal=1)
    for i in range(n):
        qi, ki = q[:, i], k[:, i]
        attn = ((qi @ ki.transpose(-1, -2)) * decay[:, i]).masked_fill(strict, 0)
        v_new = u[:, i] - w[:, i] @ state
        out[:, i] = (qi * g[:, i, :, None].exp()) @ state + attn @ v_new
        state = state * g[:, i, -1, None, None].exp() + (ki * (g[:, i, -1, None] - g[:, i]).exp()[..., None]).transpose(-1, -2) @ v_new
    return out.reshape(H, n * chunk, dv)[:, :T].transpose(0, 1).to(dt)


def recurrent_gated_delta_rule(q, k, v, g, beta):
    """Token-by-token form of the same rule (the oracle of the chunked one)."""
    q = _l2norm(q.float()) * q.shape[-1] ** -0.5
    k = _l2norm(k.float())
    T, H, dk = k.shape
    state = q.new_zeros((H, dk, v.shape[-1]))
    out = []
    for t in range(T):
        state = state * g[t].float().exp()[:, None, None]
        delta = (v[t].float() - torch.einsum("hk,hkv->hv", k[t], state)) * beta[t].float()[:, None]
        state = state + k[t][:, :, None] * delta[:, None, :]
        out.append(torch.einsum("hk,hkv->hv", q[t], state))
    return torch.stack(out).to(v.dtype)


class GatedDeltaNet(nn.Module):
    def __init__(self, cfg: Qwen35Config, layer_idx: int):
        super().__init__()
        self.layer_idx = layer_idx
        self.hk, self.hv = cfg.linear_num_key_heads, cfg.linear_num_value_heads
        self.dk, self.dv = cfg.linear_key_head_dim, cfg.linear_value_head_dim
        self.key_dim, self.value_dim = self.hk * self.dk, self.hv * self.dv
        self.kernel = cfg.linear_conv_kernel_dim
        conv_dim = 2 * self.key_dim + self.value_dim
        self.conv1d = nn.Conv1d(conv_dim, conv_dim, self.kernel, groups=conv_dim, padding=self.kernel - 1, bias=False)
        self.dt_bias = nn.Parameter(torch.ones(self.hv))
        self.A_log = nn.Parameter(torch.log(torch.empty(self.hv).uniform_(0, 16)))
        self.norm = nn.Module()
        self.norm.weight = nn.Parameter(torch.ones(self.dv))
        self.eps = cfg.rms_norm_eps
        self.out_proj = nn.Linear(self.value_dim, cfg.hidden_size, bias=False)
        self.in_proj_qkv = nn.Linear(cfg.hidden_size, conv_dim, bias=False)
        self.in_proj_z = nn.Linear(cfg.hidden_size, self.value_dim, bias=False)
        self.in_proj_b = nn.Linear(cfg.hidden_size, self.hv, bias=False)
        self.in_proj_a = nn.Linear(cfg.hidden_size, self.hv, bias=False)
        self.linear_attn_cp = getattr(cfg, "linear_attn_cp", "auto")

    def forward(self, x: torch.Tensor, ctx: PackedContext) -> torch.Tensor:
        T = x.shape[0]
        w_all = torch.cat([_w(self.in_proj_qkv.weight), _w(self.in_proj_z.weight), _w(self.in_proj_b.weight), _w(self.in_proj_a.weight)], 0)
        pad = (-w_all.shape[0]) % 8
        if pad:
            w_all = F.pad(w_all, (0, 0, 0, pad))
        proj = gemm_ops.linear(x, w_all, None)
        c = 2 * self.key_dim + self.value_dim
        mixed, z = proj[:, :c], proj[:, c:c + self.value_dim]
        b, a = proj[:, c + self.value_dim:c + self.value_dim + self.hv], proj[:, c + self.value_dim + self.hv:c + self.value_dim + 2 * self.hv]
        A_log, dt_bias, conv_w = self.A_log, self.dt_bias, self.conv1d.weight[:, 0]
        hk, hv = self.hk, self.hv
        if getattr(ctx, "kv_cache", None) is not None:
            assert ctx.sp_size == 1, "generation runs without sequence parallelism"
            return self._finish(self._forward_cached(mixed, a, b, conv_w, ctx.kv_cache), z, x, T)
        by_state = ctx.sp_size > 1 and self.cp_mode(ctx.sp_size) == "state"
        if by_state:
            return self._finish(self._forward_state_cp(mixed, a, b, conv_w, ctx, x.device), z, x, T)
        if ctx.sp_size > 1:
            # Ulysses: the convolution and the rule run on whole sequences of this rank's heads.  Heads are
            # independent (the convolution is depthwise), so one exchange in and one out carry the layer.
            n, r = ctx.sp_size, dist.get_rank(ctx.sp_group)
            assert hk % n == 0 and hv % n == 0, "linear-attention heads must divide the sequence-parallel size"
            qh, kh, vh = torch.split(mixed, [self.key_dim, self.key_dim, self.value_dim], -1)
            qh = sp.gather_seq_scatter_heads(qh.reshape(T, hk, self.dk), ctx.sp_group)
            kh = sp.gather_seq_scatter_heads(kh.reshape(T, hk, self.dk), ctx.sp_group)
            vh = sp.gather_seq_scatter_heads(vh.reshape(T, hv, self.dv), ctx.sp_group)
            ab = sp.gather_seq_scatter_heads(torch.stack([a, b], -1).float(), ctx.sp_group)
            a, b = ab[..., 0], ab[..., 1]
            hk, hv = hk // n, hv // n
            mixed = torch.cat([qh.flatten(1), kh.flatten(1), vh.flatten(1)], -1)
            rows = torch.cat([torch.arange(r * hk * self.dk, (r + 1) * hk * self.dk),
                              self.key_dim + torch.arange(r * hk * self.dk, (r + 1) * hk * self.dk),
                              2 * self.key_dim + torch.arange(r * hv * self.dv, (r + 1) * hv * self.dv)]).to(conv_w.device)
            conv_w = conv_w.index_select(0, rows)
            A_log, dt_bias = A_log[r * hv:(r + 1) * hv], dt_bias[r * hv:(r + 1) * hv]
        beta = b.sigmoid()
        g = -A_log.float().exp() * F.softplus(a.float() + dt_bias)
        plan = gdn_ops.plan_for(ctx, x.device)
        lengths, pos_in_doc, chunks = plan
        live = int(pos_in_doc.numel())  # rows after it are the padding of a sequence-parallel split
        # causal depthwise convolution inside every document, then SiLU
        seg = gdn_ops.causal_conv_silu_packed(mixed[:live], conv_w, pos_in_doc)
        q, k, v = torch.split(seg, [hk * self.dk, hk * self.dk, hv * self.dv], -1)
        q, k, v = q.reshape(-1, hk, self.dk), k.reshape(-1, hk, self.dk), v.reshape(-1, hv, self.dv)
        if hv // hk > 1:
            q, k = q.repeat_interleave(hv // hk, 1), k.repeat_interleave(hv // hk, 1)
        o = gdn_ops.chunk_gated_delta_rule_packed(q, k, v, g[:live], beta[:live], lengths, chunks)
        if o.shape[0] < mixed.shape[0]:
            o = torch.cat([o, o.new_zeros((mixed.shape[0] - o.shape[0], hv, self.dv))], 0)
        if ctx.sp_size > 1:
            o = sp.gather_heads_scatter_seq(o, ctx.sp_group)
        return self._finish(o, z, x, T)

    def cp_mode(self, sp_size: int) -> str:
        """How the layer runs under sequence parallelism: ``heads`` trades the token split for a head split (needs the
        head counts to divide the group), ``state`` keeps the tokens where they are and hands the recurrent state from
        rank to rank.  ``linear_attn_cp`` in the config picks one; ``auto`` takes ``heads`` when it divides."""
        mode = getattr(self, "linear_attn_cp", "auto")
        if mode == "auto":
            return "heads" if (self.hk % sp_size == 0 and self.hv % sp_size == 0) else "state"
        return mode

    def _forward_state_cp(self, mixed, a, b, conv_w, ctx, device):
        """All heads, this rank's tokens: convolution with a halo of ``kernel - 1`` rows from the previous rank, the
        rule with the state handed over between ranks."""
        lengths, pos_in_doc, chunks, first_continues, live = gdn_ops.cp_plan_for(ctx, device, ctx.sp_group)
        K = self.kernel
        halo = gdn_ops.conv_halo(mixed[:max(live, 0)] if live else mixed[:0], K - 1, ctx.sp_group)
        beta = b.sigmoid()
        g = -self.A_log.float().exp() * F.softplus(a.float() + self.dt_bias)
        if live:
            first = int(pos_in_doc[0]) if first_continues else 0
            halo_pos = torch.arange(first - (K - 1), first, device=device).clamp(min=0)
            seg = gdn_ops.causal_conv_silu_packed(torch.cat([halo, mixed[:live]], 0), conv_w, torch.cat([halo_pos, pos_in_doc]))[K - 1:]
        else:
            seg = mixed[:0] + 0.0 * halo.sum()
        q, k, v = torch.split(seg, [self.key_dim, self.key_dim, self.value_dim], -1)
        q, k, v = q.reshape(-1, self.hk, self.dk), k.reshape(-1, self.hk, self.dk), v.reshape(-1, self.hv, self.dv)
        if self.hv // self.hk > 1:
            q, k = q.repeat_interleave(self.hv // self.hk, 1), k.repeat_interleave(self.hv // self.hk, 1)
        o = gdn_ops.chunk_gated_delta_rule_cp(q, k, v, g[:live], beta[:live], lengths, first_continues, ctx.sp_group, chunks)
        if o.shape[0] < mixed.shape[0]:
            o = torch.cat([o, o.new_zeros((mixed.shape[0] - o.shape[0], self.hv, self.dv))], 0)
        return o

    def _forward_cached(self, mixed, a, b, conv_w, cache):
        """Generation: every sequence continues from its stored convolution tail (the last ``kernel - 1`` rows that went
        into the convolution) and its state matrix; both are replaced by their values after this pass' tokens.  The rule
        runs on the unchanged chunk scan with the state entering and leaving through ``scan_with_state``."""
        K, dev = self.kernel, mixed.device
        store = cache.state.setdefault(self.layer_idx, {})
        beta = b.sigmoid()
        g = -self.A_log.float().exp() * F.softplus(a.float() + self.dt_bias)
        rep = self.hv // self.hk
        outs, at = [], 0
        for i, n in enumerate(cache.new_lens):
            if n == 0:
                continue
            have = cache.had[i]
            tail, S = store.get(i, (mixed.new_zeros((K - 1, mixed.shape[1])), None))
            rows = torch.cat([tail, mixed[at:at + n]], 0)
            pos = torch.arange(have - (K - 1), have + n, device=dev).clamp(min=0)
            seg = gdn_ops.causal_conv_silu_packed(rows, conv_w, pos)[K - 1:]
            q, k, v = torch.split(seg, [self.key_dim, self.key_dim, self.value_dim], -1)
            q, k, v = q.reshape(n, self.hk, self.dk), k.reshape(n, self.hk, self.dk), v.reshape(n, self.hv, self.dv)
            if rep > 1:
                q, k = q.repeat_interleave(rep, 1), k.repeat_interleave(rep, 1)
            o, S = gdn_ops.chunk_gated_delta_rule_stateful(q, k, v, g[at:at + n], beta[at:at + n], S)
            store[i] = (rows[-(K - 1):].detach(), S.detach())
            outs.append(o)
            at += n
        return torch.cat(outs, 0)

    def _finish(self, o, z, x, T):
        # RMSNorm over the head dim, gated by SiLU(z)
        o = norm_ops.rmsnorm(o.reshape(-1, self.dv).to(x.dtype), self.norm.weight, self.eps)
        o = (o.float() * F.silu(z.reshape(-1, self.dv).float())).to(x.dtype).reshape(T, self.value_dim)
        return gemm_ops.linear(o, _w(self.out_proj.weight), None)


class GatedAttention(nn.Module):
    """Softmax attention whose query projection also emits a per-channel output gate; q/k RMSNorm; partial rotary."""

    def __init__(self, cfg: Qwen35Config, layer_idx: int):
        super().__init__()
        self.cfg, self.layer_idx = cfg, layer_idx
        H, D = cfg.hidden_size, cfg.head_dim
        self.n_q, self.n_kv, self.head_dim = cfg.num_attention_heads, cfg.num_key_value_heads, D
        self.q_proj = nn.Linear(H, self.n_q * D * 2, bias=cfg.attention_bias)
        self.k_proj = nn.Linear(H, self.n_kv * D, bias=cfg.attention_bias)
        self.v_proj = nn.Linear(H, self.n_kv * D, bias=cfg.attention_bias)
        self.o_proj = nn.Linear(self.n_q * D, H, bias=cfg.attention_bias)
        self.q_norm, self.k_norm = ZRMSNorm(D, cfg.rms_norm_eps), ZRMSNorm(D, cfg.rms_norm_eps)

    def forward(self, x, ctx: PackedContext):
        T, D = x.shape[0], self.head_dim
        qg = gemm_ops.linear(x, _w(self.q_proj.weight), _w(self.q_proj.bias)).view(T, self.n_q, 2 * D)
        q, gate = qg[..., :D], qg[..., D:].reshape(T, self.n_q * D)
        k = gemm_ops.linear(x, _w(self.k_proj.weight), _w(self.k_proj.bias)).view(T, self.n_kv, D)
        v = gemm_ops.linear(x, _w(self.v_proj.weight), _w(self.v_proj.bias)).view(T, self.n_kv, D)
        q = self.q_norm(q.reshape(-1, D)).view(T, self.n_q, D)
        k = self.k_norm(k.reshape(-1, D)).view(T, self.n_kv, D)
        if ctx.sp_size > 1:  # Ulysses: trade the sequence split for a head split around attention
            q, k, v = sp.seq_to_head_qkv(q, k, v, ctx.sp_group)
        q, k = rope_ops.rope_apply(q, ctx.cos, ctx.sin), rope_ops.rope_apply(k, ctx.cos, ctx.sin)
        if getattr(ctx, "kv_cache", None) is not None:  # generation: new tokens against the cached rows of their sequence
            assert ctx.sp_size == 1, "generation runs without sequence parallelism"
            k_all, v_all, cu_k, max_k = ctx.kv_cache.extend(self.layer_idx, k, v.contiguous())
            o = attn_ops.varlen_attn(q, k_all, v_all, ctx.cu_seqlens, cu_k, ctx.max_seqlen, max_k, causal=ctx.causal,
                                     softmax_scale=1.0 / math.sqrt(D))
        else:
            o = attn_ops.varlen_attn(q, k, v, ctx.cu_seqlens, ctx.cu_seqlens, ctx.max_seqlen, ctx.max_seqlen, causal=ctx.causal,
                                     softmax_scale=1.0 / math.sqrt(D))
        if ctx.sp_size > 1:
            o = sp.head_to_seq(o, ctx.sp_group, self.n_q, self.n_kv)
        o = (o.reshape(T, -1).float() * torch.sigmoid(gate.float())).to(x.dtype)
        return gemm_ops.linear(o, _w(self.o_proj.weight), _w(self.o_proj.bias))


class Qwen35Layer(nn.Module):
    def __init__(self, cfg: Qwen35Config, layer_idx: int):
        super().__init__()
        self.layer_type = cfg.layer_types[layer_idx]
        if self.layer_type == "linear_attention":
            self.linear_attn = GatedDeltaNet(cfg, layer_idx)
        else:
            self.self_attn = GatedAttention(cfg, layer_idx)
        self.mlp = SwiGLUMLP(cfg.hidden_size, cfg.intermediate_size)
        self.input_layernorm = ZRMSNorm(cfg.hidden_size, cfg.rms_norm_eps)
        self.post_attention_layernorm = ZRMSNorm(cfg.hidden_size, cfg.rms_norm_eps)

    def forward(self, h, residual, ctx: PackedContext):
        if residual is None:
            residual, x = h, self.input_layernorm(h)
        else:
            x, residual = self.input_layernorm(h, residual)
        a = self.linear_attn(x, ctx) if self.layer_type == "linear_attention" else self.self_attn(x, ctx)
        x, residual = self.post_attention_layernorm(a, residual)
        out = self.mlp(x)
        if isinstance(out, tuple):  # sparse blocks also return router statistics
            ctx.aux.append(out[1])
            out = out[0]
        return out, residual


class Qwen35Backbone(DecoderBackbone):
    layer_cls = Qwen35Layer

    def __init__(self, cfg: Qwen35Config):
        super().__init__(cfg)
        self.norm = ZRMSNorm(cfg.hidden_size, cfg.rms_norm_eps)
        self.rot_dim = int(cfg.head_dim * cfg.partial_rotary_factor)
        self.register_buffer("inv_freq", rope_ops.inv_freq(self.rot_dim, cfg.rope_theta), persistent=False)

    def rope_tables(self, position_ids: torch.Tensor):
        cfg = self.cfg
        invf = self.inv_freq
        if invf.dtype != torch.float32 or invf.device != position_ids.device:
            invf = rope_ops.inv_freq(self.rot_dim, cfg.rope_theta, device=position_ids.device)
        mode = {"none": rope_ops.MODE_PLAIN, "sectioned": rope_ops.MODE_SECTIONED, "interleaved": rope_ops.MODE_INTERLEAVED}[
            cfg.mrope_mode if position_ids.dim() == 2 else "none"]
        sections = tuple(cfg.mrope_section) if (cfg.mrope_section and mode != rope_ops.MODE_PLAIN) else (0, 0, 0)
        return rope_ops.rope_table(position_ids, invf, mode, sections)


class Qwen35LM(DecoderLM):
    supports_kv_cache = True  # attention layers cache keys / values, linear-attention layers their convolution tail and state
    config_class = Qwen35Config
    backbone_cls = Qwen35Backbone
    _no_split_modules = ["Qwen35Layer"]

    def _init_weights(self, m):
        super()._init_weights(m)
        if isinstance(m, ZRMSNorm):
            nn.init.zeros_(m.weight)

    def convert_hf_state_dict(self, sd):
        out = {}
        for k, v in sd.items():
            k = k.replace("model.language_model.", "model.")
            if k.startswith(("model.visual.", "mtp.")):  # text-only use of a multimodal checkpoint; multi-token-prediction head
                continue
            out[k] = v
        return out


# ------------------------------------------------------------------------------- mixture-of-experts variant
from .moe_lm import MoEConfig, MoEDecoderLM, SparseMoeBlock  # noqa: E402


@dataclass
class Qwen35MoEConfig(MoEConfig, Qwen35Config):
    """``qwen3_5_moe_text``: the hybrid layer pattern with sparse MLPs (routed experts + sigmoid-gated shared expert)."""

    model_type: str = "qwen3_5_moe_text"

    @classmethod
    def from_dict(cls, d):
        d = dict(d.get("text_config") or d)
        rope = d.get("rope_parameters") or d.get("rope_scaling") or {}
        if "partial_rotary_factor" in rope:
            d["partial_rotary_factor"] = rope["partial_rotary_factor"]  # the rope dict is what the hub model reads
        return MoEConfig.from_dict.__func__(cls, d)


class Qwen35MoELayer(Qwen35Layer):
    def __init__(self, cfg, layer_idx: int):
        super().__init__(cfg, layer_idx)
        if cfg.is_sparse_layer(layer_idx):
            self.mlp = SparseMoeBlock(cfg)


class Qwen35MoEBackbone(Qwen35Backbone):
    layer_cls = Qwen35MoELayer


class Qwen35MoELM(MoEDecoderLM):
    config_class = Qwen35MoEConfig
    backbone_cls = Qwen35MoEBackbone
    _no_split_modules = ["Qwen35MoELayer"]

    def _init_weights(self, m):
        super()._init_weights(m)
        if isinstance(m, ZRMSNorm):
            nn.init.zeros_(m.weight)
