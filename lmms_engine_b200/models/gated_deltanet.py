"""``gated_deltanet``: a decoder made only of Gated-DeltaNet linear-attention blocks, in the configuration and
checkpoint layout of the FLA library (the reference builds it from that library's registry,
src/lmms_engine/mapping_func.py:18-21, examples/dgn/train_dgn_1b.yaml).

Block: RMSNorm -> linear attention -> RMSNorm -> SwiGLU MLP with fused residual adds.  Linear attention: separate
q / k / v projections each followed by a short causal depthwise convolution + SiLU inside the document, L2-normalised
q / k, decay ``g = -exp(A_log) * softplus(a + dt_bias)``, write strength ``beta = sigmoid(b)`` (doubled when negative
eigenvalues are allowed), the chunked gated delta rule of ``ops/gdn.py`` (state recurrence in CUDA kernels), an output
RMSNorm gated by ``SiLU(g_proj(x))`` per head, and the output projection.  Value heads may outnumber key heads
(keys / queries are repeated).  Softmax-attention layers mixed in through ``attn`` are not built.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import gdn as gdn_ops
from ..ops import gemm as gemm_ops
from ..ops import norm as norm_ops
from .decoder_lm import DecoderBackbone, DecoderConfig, DecoderLM, PackedContext, RMSNorm, SwiGLUMLP, _w


@dataclass
class GatedDeltaNetConfig(DecoderConfig):
    model_type: str = "gated_deltanet"
    hidden_size: int = 2048
    num_hidden_layers: int = 21
    num_heads: int = 6
    num_v_heads: Optional[int] = None
    head_dim: int = 256
    expand_v: float = 2.0
    conv_size: int = 4
    use_gate: bool = True
    use_short_conv: bool = True
    allow_neg_eigval: bool = False
    hidden_ratio: Optional[int] = 4
    norm_eps: float = 1e-6
    vocab_size: int = 32000

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "GatedDeltaNetConfig":
        d = dict(d)
        if d.get("attn"):
            raise NotImplementedError("gated_deltanet: softmax-attention layers mixed in through `attn` are not built")
        d.pop("attn", None)
        d["model_type"] = "gated_deltanet"
        hidden = int(d.get("hidden_size", 2048))
        if d.get("intermediate_size") is None:
            # a multiple of 256 next to 2/3 * hidden_ratio * hidden, as the library sizes its gated MLP
            ratio = d.get("hidden_ratio") or 4
            d["intermediate_size"] = 256 * ((int(hidden * ratio * 2 / 3) + 255) // 256)
        d.setdefault("num_attention_heads", int(d.get("num_heads", 6)))
        d.setdefault("num_key_value_heads", int(d.get("num_heads", 6)))
        d["rms_norm_eps"] = float(d.get("norm_eps", 1e-6))
        return super().from_dict(d)

    def to_dict(self) -> Dict[str, Any]:
        d = super().to_dict()
        d["architectures"] = ["GatedDeltaNetForCausalLM"]
        return d


class FlaGatedDeltaNet(nn.Module):
    def __init__(self, cfg: GatedDeltaNetConfig, layer_idx: int):
        super().__init__()
        self.hk = cfg.num_heads
        self.hv = cfg.num_v_heads or cfg.num_heads
        self.dk = cfg.head_dim
        self.dv = int(cfg.head_dim * cfg.expand_v)
        self.key_dim, self.value_dim = self.hk * self.dk, self.hv * self.dv
        self.use_gate, self.use_conv, self.neg = cfg.use_gate, cfg.use_short_conv, cfg.allow_neg_eigval
        self.eps = cfg.norm_eps
        H = cfg.hidden_size
        self.q_proj = nn.Linear(H, self.key_dim, bias=False)
        self.k_proj = nn.Linear(H, self.key_dim, bias=False)
        self.v_proj = nn.Linear(H, self.value_dim, bias=False)
        self.a_proj = nn.Linear(H, self.hv, bias=False)
        self.b_proj = nn.Linear(H, self.hv, bias=False)
        self.A_log = nn.Parameter(torch.log(torch.empty(self.hv).uniform_(0, 16)))
        dt = torch.exp(torch.rand(self.hv) * (torch.log(torch.tensor(0.1)) - torch.log(torch.tensor(0.001))) + torch.log(torch.tensor(0.001)))
        dt = dt.clamp(min=1e-4)
        self.dt_bias = nn.Parameter(dt + torch.log(-torch.expm1(-dt)))
        if self.use_conv:
            for name, dim in (("q_conv1d", self.key_dim), ("k_conv1d", self.key_dim), ("v_conv1d", self.value_dim)):
                conv = nn.Module()
                conv.weight = nn.Parameter(torch.empty(dim, 1, cfg.conv_size).uniform_(-cfg.conv_size ** -0.5, cfg.conv_size ** -0.5))
                setattr(self, name, conv)
        if self.use_gate:
            self.g_proj = nn.Linear(H, self.value_dim, bias=False)
        self.o_norm = nn.Module()
        self.o_norm.weight = nn.Parameter(torch.ones(self.dv))
        self.o_proj = nn.Linear(self.value_dim, H, bias=False)

    def forward(self, x: torch.Tensor, ctx: PackedContext) -> torch.Tensor:
        T = x.shape[0]
        parts = [self.q_proj, self.k_proj, self.v_proj, self.a_proj, self.b_proj] + ([self.g_proj] if self.use_gate else [])
        w_all = torch.cat([_w(p.weight) for p in parts], 0)
        pad = (-w_all.shape[0]) % 8
        if pad:
            w_all = F.pad(w_all, (0, 0, 0, pad))
        proj = gemm_ops.linear(x, w_all, None)
        sizes = [self.key_dim, self.key_dim, self.value_dim, self.hv, self.hv] + ([self.value_dim] if self.use_gate else [])
        cols = torch.split(proj[:, : sum(sizes)], sizes, -1)
        q, k, v, a, b = cols[:5]
        lengths, pos_in_doc, chunks = gdn_ops.plan_for(ctx, x.device)
        live = int(pos_in_doc.numel())
        if self.use_conv:
            w = torch.cat([self.q_conv1d.weight, self.k_conv1d.weight, self.v_conv1d.weight], 0)[:, 0]
            mixed = gdn_ops.causal_conv_silu_packed(torch.cat([q, k, v], -1)[:live], w, pos_in_doc)
            q, k, v = torch.split(mixed, [self.key_dim, self.key_dim, self.value_dim], -1)
        else:
            q, k, v = F.silu(q[:live]), F.silu(k[:live]), F.silu(v[:live])
        q, k, v = q.reshape(-1, self.hk, self.dk), k.reshape(-1, self.hk, self.dk), v.reshape(-1, self.hv, self.dv)
        if self.hv // self.hk > 1:
            q, k = q.repeat_interleave(self.hv // self.hk, 1), k.repeat_interleave(self.hv // self.hk, 1)
        beta = b[:live].float().sigmoid() * (2.0 if self.neg else 1.0)
        g = -self.A_log.float().exp() * F.softplus(a[:live].float() + self.dt_bias)
        o = gdn_ops.chunk_gated_delta_rule_packed(q, k, v, g, beta, lengths, chunks)
        if o.shape[0] < T:
            o = torch.cat([o, o.new_zeros((T - o.shape[0], self.hv, self.dv))], 0)
        o = norm_ops.rmsnorm(o.reshape(-1, self.dv).to(x.dtype), self.o_norm.weight, self.eps)
        if self.use_gate:
            o = (o.float() * F.silu(cols[5].reshape(-1, self.dv).float())).to(x.dtype)
        return gemm_ops.linear(o.reshape(T, self.value_dim), _w(self.o_proj.weight), None)


class GatedDeltaNetBlock(nn.Module):
    def __init__(self, cfg: GatedDeltaNetConfig, layer_idx: int):
        super().__init__()
        self.attn_norm = RMSNorm(cfg.hidden_size, cfg.norm_eps)
        self.attn = FlaGatedDeltaNet(cfg, layer_idx)
        self.mlp_norm = RMSNorm(cfg.hidden_size, cfg.norm_eps)
        self.mlp = SwiGLUMLP(cfg.hidden_size, cfg.intermediate_size)

    def forward(self, h, residual, ctx: PackedContext):
        if residual is None:
            residual, x = h, self.attn_norm(h)
        else:
            x, residual = self.attn_norm(h, residual)
        x, residual = self.mlp_norm(self.attn(x, ctx), residual)
        return self.mlp(x), residual


class GatedDeltaNetBackbone(DecoderBackbone):
    layer_cls = GatedDeltaNetBlock


class GatedDeltaNetLM(DecoderLM):
    supports_kv_cache = False
    config_class = GatedDeltaNetConfig
    backbone_cls = GatedDeltaNetBackbone
    _no_split_modules = ["GatedDeltaNetBlock"]

    # the library names the embedding table ``model.embeddings``
    def convert_hf_state_dict(self, sd):
        return {("model.embed_tokens.weight" if k == "model.embeddings.weight" else k): v for k, v in sd.items()}

    def export_hf_state_dict(self, sd):
        return {("model.embeddings.weight" if k == "model.embed_tokens.weight" else k): v for k, v in sd.items()}
