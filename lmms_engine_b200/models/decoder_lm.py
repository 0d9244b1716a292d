"""Packed-varlen dense decoder LM (Qwen2 / Qwen2.5 / Qwen3 families).

The model is varlen-first: tokens of all documents of a step form one flat ``[T]`` stream
with ``cu_seqlens`` boundaries and per-document ``position_ids``; there is no padded
``[B, L]`` tensor anywhere inside.  Padded HF-style batches (``input_ids [n, L]`` +
``attention_mask``) are accepted at the door and unpadded once.  Parameter names and
shapes are those of the HF checkpoints (``model.layers.N.self_attn.q_proj.weight`` ...),
so safetensors load/save and merged checkpoints stay interchangeable.

What this replaces in the reference: the monkey-patched HF forwards for rmpad + Liger +
Ulysses, i.e. src/lmms_engine/models/qwen2/qwen2_ops.py:61-310 (model / layer / attention
forward), src/lmms_engine/models/qwen2/qwen2_liger.py:27-176 (per-document label shift +
fused linear-CE + SP loss gather), src/lmms_engine/models/qwen3/qwen3_ops.py:237-297
(QK-RMSNorm), src/lmms_engine/models/sequence_packing_utils.py:10-62 (unpad).
"""
from __future__ import annotations

import math
from dataclasses import asdict, dataclass, field, fields
from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint

from ..ops import attention as attn_ops
from ..ops import cross_entropy as ce_ops
from ..ops import gemm as gemm_ops
from ..ops import norm as norm_ops
from ..ops import rope as rope_ops
from ..ops import swiglu as swiglu_ops
from ..parallel import fused_ops, tp_ops
from ..parallel.sequence_parallel import ulysses as sp

IGNORE_INDEX = -100


def _w(p):
    """Plain local tensor of a parameter (tensor-parallel parameters are DTensors on the tp mesh)."""
    if p is None:
        return None
    return p.to_local() if hasattr(p, "to_local") else p


@dataclass
class DecoderConfig:
    model_type: str = "qwen2"
    vocab_size: int = 151936
    hidden_size: int = 3584
    intermediate_size: int = 18944
    num_hidden_layers: int = 28
    num_attention_heads: int = 28
    num_key_value_heads: int = 4
    head_dim: Optional[int] = None
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e6
    tie_word_embeddings: bool = False
    attention_bias: Optional[bool] = None  # None: by family (qwen2 True, qwen3 False)
    qk_norm: Optional[bool] = None  # None: by family (qwen3 True)
    sliding_window: Optional[int] = None
    use_sliding_window: bool = False
    max_position_embeddings: int = 32768
    initializer_range: float = 0.02
    hidden_act: str = "silu"
    torch_dtype: str = "bfloat16"
    architectures: Optional[List[str]] = None
    # multimodal rope (used by the VL wrappers): "none" | "sectioned" | "interleaved"
    mrope_mode: str = "none"
    mrope_section: Optional[List[int]] = None
    extra: Dict[str, Any] = field(default_factory=dict)

    def __post_init__(self):
        if self.head_dim is None:
            self.head_dim = self.hidden_size // self.num_attention_heads
        if self.attention_bias is None:
            self.attention_bias = self.model_type.startswith("qwen2")
        if self.qk_norm is None:
            self.qk_norm = self.model_type.startswith("qwen3")
        if self.architectures is None:
            self.architectures = [{"qwen2": "Qwen2ForCausalLM", "qwen3": "Qwen3ForCausalLM"}.get(self.model_type, "Qwen2ForCausalLM")]

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "DecoderConfig":
        d = dict(d)
        rope = d.pop("rope_parameters", None) or d.pop("rope_scaling", None)
        known = {f.name for f in fields(cls)}
        kw = {k: v for k, v in d.items() if k in known}
        extra = {k: v for k, v in d.items() if k not in known}
        if isinstance(rope, dict):
            if "rope_theta" in rope and "rope_theta" not in kw:
                kw["rope_theta"] = rope["rope_theta"]
            if rope.get("mrope_section"):
                kw.setdefault("mrope_section", list(rope["mrope_section"]))
                kw.setdefault("mrope_mode", "interleaved" if rope.get("mrope_interleaved") else "sectioned")
        if "dtype" in extra and "torch_dtype" not in kw:
            kw["torch_dtype"] = str(extra.pop("dtype")).replace("torch.", "")
        kw["extra"] = {**kw.get("extra", {}), **extra}
        return cls(**kw)

    def to_dict(self) -> Dict[str, Any]:
        d = asdict(self)
        extra = d.pop("extra")
        d.pop("qk_norm")
        d.pop("mrope_mode")
        sect = d.pop("mrope_section")
        if sect:
            d["rope_scaling"] = {"type": "default", "mrope_section": sect, "mrope_interleaved": self.mrope_mode == "interleaved"}
        d.update(extra)
        return d


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def forward(self, x, residual=None):
        return norm_ops.rmsnorm(x, self.weight, self.eps, 0.0, residual)


class Attention(nn.Module):
    def __init__(self, cfg: DecoderConfig, layer_idx: int):
        super().__init__()
        self.cfg = cfg
        self.layer_idx = layer_idx
        H, D = cfg.hidden_size, cfg.head_dim
        self.n_q, self.n_kv, self.head_dim = cfg.num_attention_heads, cfg.num_key_value_heads, D
        self.q_proj = nn.Linear(H, self.n_q * D, bias=cfg.attention_bias)
        self.k_proj = nn.Linear(H, self.n_kv * D, bias=cfg.attention_bias)
        self.v_proj = nn.Linear(H, self.n_kv * D, bias=cfg.attention_bias)
        self.o_proj = nn.Linear(self.n_q * D, H, bias=False)
        if cfg.qk_norm:
            self.q_norm = RMSNorm(D, cfg.rms_norm_eps)
            self.k_norm = RMSNorm(D, cfg.rms_norm_eps)
        window = cfg.sliding_window if (cfg.use_sliding_window and cfg.sliding_window) else None
        self.window = (window, -1) if window else (-1, -1)

    def forward(self, x: torch.Tensor, ctx: "PackedContext") -> torch.Tensor:
        D = self.head_dim
        # one GEMM for q, k, v: the three weights are concatenated on the fly (tens of MB,
        # microseconds) so the projection runs as a single [T, (Hq+2Hkv)D] product
        w = torch.cat([_w(self.q_proj.weight), _w(self.k_proj.weight), _w(self.v_proj.weight)], 0)
        b = (torch.cat([_w(self.q_proj.bias), _w(self.k_proj.bias), _w(self.v_proj.bias)], 0)
             if self.q_proj.bias is not None else None)
        nq, nkv = self.n_q * D, self.n_kv * D
        # fused collectives: the projection kernels move the data between the ranks themselves
        fc_tp = fused_ops.context_for(ctx.tp_group) if (ctx.tp_size > 1 and x.is_cuda and fused_ops.tp_supported(x.shape[0])) else None
        fc_sp = (fused_ops.context_for(ctx.sp_group)
                 if (ctx.sp_size > 1 and x.is_cuda and fused_ops.ulysses_supported(self.n_q, self.n_kv, D, ctx.sp_size)) else None)
        if fc_sp is not None:
            q, k, v = fused_ops.ulysses_qkv(x, w, b, fc_sp, self.n_q, self.n_kv, D, self.layer_idx)
        else:
            if fc_tp is not None:
                qkv = fused_ops.column_linear(x, w, b, fc_tp)
            else:
                if ctx.tp_size > 1:
                    # sequence-parallel tensor parallelism: gather the token shards, project onto this
                    # rank's heads; the row-parallel output projection below reduce-scatters back
                    x = tp_ops.all_gather_tokens(x, ctx.tp_group)
                qkv = gemm_ops.linear(x, w, b)
            T = qkv.shape[0]
            q = qkv[:, :nq].view(T, self.n_q, D)
            k = qkv[:, nq : nq + nkv].view(T, self.n_kv, D)
            v = qkv[:, nq + nkv :].view(T, self.n_kv, D)
        if self.cfg.qk_norm:  # per head, so it commutes with the head exchange
            q = self.q_norm(q.reshape(-1, D)).view(q.shape)
            k = self.k_norm(k.reshape(-1, D)).view(k.shape)
        if ctx.sp_size > 1 and fc_sp is None:
            # Ulysses: trade the sequence split for a head split around attention
            q, k, v = sp.seq_to_head_qkv(q, k, v, ctx.sp_group)
        k_plain = k
        q = rope_ops.rope_apply(q, ctx.cos, ctx.sin)
        k = rope_ops.rope_apply(k, ctx.cos, ctx.sin)
        if getattr(self, "nsa", None) is not None:
            # native sparse attention (added to a built model by the "nsa" patch of the bagel family)
            assert ctx.sp_size == 1 and ctx.tp_size == 1, "native sparse attention runs without sequence / tensor parallelism"
            from ..ops import nsa as nsa_ops

            k_cmp, counts = nsa_ops.compress(k_plain, self.compress_key, ctx.cu_seqlens, self.nsa.kernel_size,
                                             self.nsa.kernel_stride, self.intra_block_pe, self.nsa.compress_type)
            v_cmp, _ = nsa_ops.compress(v, self.compress_value, ctx.cu_seqlens, self.nsa.kernel_size,
                                        self.nsa.kernel_stride, None, self.nsa.compress_type)
            gates = torch.sigmoid(gemm_ops.linear(x, _w(self.g_proj.weight), None)).view(x.shape[0], self.n_q, 3)
            o = nsa_ops.nsa_attention(q, k, v, k_cmp, v_cmp, counts, gates, ctx.cu_seqlens, self.nsa, 1.0 / math.sqrt(D))
        elif getattr(ctx, "kv_cache", None) is not None:
            # generation: the new tokens attend to the cached rows of their sequence and to themselves
            assert ctx.sp_size == 1 and ctx.tp_size == 1, "the key / value cache runs without sequence / tensor parallelism"
            k_all, v_all, cu_k, max_k = ctx.kv_cache.extend(self.layer_idx, k, v)
            o = attn_ops.varlen_attn(q, k_all, v_all, ctx.cu_seqlens, cu_k, ctx.max_seqlen, max_k, causal=ctx.causal,
                                     softmax_scale=1.0 / math.sqrt(D), window_size=self.window)
        else:
            o = attn_ops.varlen_attn(
                q, k, v, ctx.cu_seqlens, ctx.cu_seqlens, ctx.max_seqlen, ctx.max_seqlen, causal=ctx.causal,
                softmax_scale=1.0 / math.sqrt(D), window_size=self.window,
            )
        if fc_sp is not None:
            return fused_ops.ulysses_out(o, _w(self.o_proj.weight), fc_sp, self.n_q, D, self.layer_idx)
        if ctx.sp_size > 1:
            o = sp.head_to_seq(o, ctx.sp_group, self.n_q, self.n_kv)
        if fc_tp is not None:
            return fused_ops.row_linear(o.reshape(o.shape[0], -1), _w(self.o_proj.weight), fc_tp)
        out = gemm_ops.linear(o.reshape(o.shape[0], -1), _w(self.o_proj.weight), None)
        if ctx.tp_size > 1:
            out = tp_ops.reduce_scatter_tokens(out, ctx.tp_group)
        return out


class SwiGLUMLP(nn.Module):
    def __init__(self, hidden: int, inter: int):
        super().__init__()
        self.gate_proj = nn.Linear(hidden, inter, bias=False)
        self.up_proj = nn.Linear(hidden, inter, bias=False)
        self.down_proj = nn.Linear(inter, hidden, bias=False)

        self.tp_group = None

    def forward(self, x):
        if self.tp_group is not None and x.is_cuda and fused_ops.tp_supported(x.shape[0]):
            fc = fused_ops.context_for(self.tp_group)
            if fc is not None:
                # all-gather -> [gate; up] GEMM, GEMM -> reduce-scatter: two kernels carry both collectives
                wg, wu = _w(self.gate_proj.weight), _w(self.up_proj.weight)
                gu = fused_ops.column_linear(x, torch.cat([wg, wu], 0), None, fc)
                h = swiglu_ops.swiglu(gu[:, : wg.shape[0]], gu[:, wg.shape[0] :])
                return fused_ops.row_linear(h, _w(self.down_proj.weight), fc)
        if self.tp_group is not None:
            x = tp_ops.all_gather_tokens(x, self.tp_group)
        y = swiglu_ops.swiglu_mlp(x, _w(self.gate_proj.weight), _w(self.up_proj.weight), _w(self.down_proj.weight))
        if self.tp_group is not None:
            y = tp_ops.reduce_scatter_tokens(y, self.tp_group)
        return y


class DecoderLayer(nn.Module):
    def __init__(self, cfg: DecoderConfig, layer_idx: int):
        super().__init__()
        self.self_attn = Attention(cfg, layer_idx)
        self.mlp = self.build_mlp(cfg, layer_idx)
        self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps)
        self.post_attention_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps)

    def build_mlp(self, cfg, layer_idx):
        return SwiGLUMLP(cfg.hidden_size, cfg.intermediate_size)

    def forward(self, h, residual, ctx: "PackedContext"):
        """``h`` is the output of the previous block, ``residual`` the running stream
        (``None`` for the first layer).  Returns the MLP output and the updated stream."""
        if residual is None:
            residual = h
            x = self.input_layernorm(h)
        else:
            x, residual = self.input_layernorm(h, residual)
        a = self.self_attn(x, ctx)
        x, residual = self.post_attention_layernorm(a, residual)
        out = self.mlp(x)
        if isinstance(out, tuple):  # MoE blocks also return router statistics
            ctx.aux.append(out[1])
            out = out[0]
        return out, residual


class PackedContext:
    """Everything a layer needs to know about the packed token stream of this step.

    Deliberately NOT a dataclass: FSDP2's ``cast_forward_inputs`` walks into dataclass arguments of every wrapped
    module, rebuilds them and casts their floating-point tensors to the parameter dtype.  That would turn the fp32
    rotary tables into bf16 behind kernels that read them as fp32, and hand every layer a copy of ``aux`` so that
    router losses appended by the layers never reach the model.  A plain object is passed through untouched."""

    def __init__(self, cu_seqlens: torch.Tensor, max_seqlen: int, cos: torch.Tensor, sin: torch.Tensor, causal: bool = True,
                 sp_group: Any = None, sp_size: int = 1, tp_group: Any = None, tp_size: int = 1, aux: Optional[List[Any]] = None,
                 deepstack: Optional[List[torch.Tensor]] = None, deepstack_index: Optional[torch.Tensor] = None,
                 split_group: Any = None, split_total: int = 0):
        self.cu_seqlens = cu_seqlens  # int32 [n_docs + 1] over the FULL (un-split) sequence
        self.max_seqlen = max_seqlen
        self.cos, self.sin = cos, sin  # fp32 [T_full, rot_dim]
        self.causal = causal
        self.sp_group, self.sp_size = sp_group, sp_size
        self.tp_group, self.tp_size = tp_group, tp_size
        self.aux = [] if aux is None else aux
        self.deepstack = deepstack  # per-layer additive visual features
        self.deepstack_index = deepstack_index
        self.split_group = split_group  # group over which the token stream is split between blocks (None: not split)
        self.split_total = split_total  # padded length of the whole stream


def unpad_batch(input_ids, attention_mask, labels=None, position_ids=None):
    """``[n, L]`` padded batch -> flat stream, ``cu_seqlens`` and per-document positions."""
    mask = attention_mask.bool()
    lens = mask.sum(-1).to(torch.int32)
    cu = F.pad(torch.cumsum(lens, 0, dtype=torch.int32), (1, 0))
    idx = torch.nonzero(mask.flatten(), as_tuple=False).flatten()
    flat_ids = input_ids.flatten()[idx]
    flat_labels = labels.flatten()[idx] if labels is not None else None
    if position_ids is None:
        pos = (torch.cumsum(mask.long(), -1) - 1).flatten()[idx]
    else:
        pos = position_ids.flatten(-2)[..., idx] if position_ids.dim() == 3 else position_ids.flatten()[idx]
    return flat_ids, flat_labels, pos, cu, idx


def shift_labels_per_document(labels: torch.Tensor, cu_seqlens: torch.Tensor) -> torch.Tensor:
    """Next-token targets that never cross a document boundary: position t gets
    ``labels[t+1]`` and the last token of every document gets ``-100``."""
    shifted = torch.roll(labels, -1, 0)
    last = (cu_seqlens[1:] - 1).long()
    # an empty leading document would give -1; the stream's last token is always a document end
    last = torch.where(last >= 0, last, torch.full_like(last, labels.shape[0] - 1))
    shifted = shifted.index_fill(0, last, IGNORE_INDEX)
    return shifted


class DecoderBackbone(nn.Module):
    layer_cls = DecoderLayer

    def __init__(self, cfg: DecoderConfig):
        super().__init__()
        self.cfg = cfg
        self.embed_tokens = nn.Embedding(cfg.vocab_size, cfg.hidden_size)
        self.layers = nn.ModuleList([self.layer_cls(cfg, i) for i in range(cfg.num_hidden_layers)])
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps)
        self.gradient_checkpointing = False
        self.register_buffer("inv_freq", rope_ops.inv_freq(cfg.head_dim, cfg.rope_theta), persistent=False)

    def rope_tables(self, position_ids: torch.Tensor):
        cfg = self.cfg
        invf = self.inv_freq
        if invf.dtype != torch.float32 or invf.device != position_ids.device:
            invf = rope_ops.inv_freq(cfg.head_dim, cfg.rope_theta, device=position_ids.device)
        mode = {"none": rope_ops.MODE_PLAIN, "sectioned": rope_ops.MODE_SECTIONED, "interleaved": rope_ops.MODE_INTERLEAVED}[
            cfg.mrope_mode if position_ids.dim() == 2 else "none"
        ]
        sections = tuple(cfg.mrope_section) if (cfg.mrope_section and mode != rope_ops.MODE_PLAIN) else (0, 0, 0)
        return rope_ops.rope_table(position_ids, invf, mode, sections)

    def forward(self, inputs_embeds: torch.Tensor, ctx: PackedContext) -> torch.Tensor:
        h, residual = inputs_embeds, None
        for i, layer in enumerate(self.layers):
            if self.gradient_checkpointing and self.training:
                h, residual = checkpoint(layer, h, residual, ctx, use_reentrant=False)
            else:
                h, residual = layer(h, residual, ctx)
            if ctx.deepstack is not None and i < len(ctx.deepstack):
                # Qwen3-VL deepstack: add visual features to the stream at visual positions
                if ctx.split_group is None:
                    h = h.index_add(0, ctx.deepstack_index, ctx.deepstack[i].to(h.dtype))
                else:
                    # the stream is split over a sequence- / tensor-parallel group while the indices address the whole
                    # sequence: scatter into a full-length buffer and keep this rank's slice (no host round trip)
                    full = h.new_zeros((ctx.split_total, h.shape[1])).index_add_(0, ctx.deepstack_index, ctx.deepstack[i].to(h.dtype))
                    h = h + sp.slice_for_rank(full, ctx.split_group)
        out, _ = self.norm(h, residual)
        return out


class DecoderLM(nn.Module):
    """Causal LM head over :class:`DecoderBackbone` with fused linear + cross-entropy."""

    config_class = DecoderConfig
    backbone_cls = DecoderBackbone
    _no_split_modules = ["DecoderLayer"]
    supports_kv_cache = True  # generation on cached keys / values (models/kv_cache.py); families with other mixers say False

    def __init__(self, cfg: DecoderConfig):
        super().__init__()
        self.config = cfg
        self.model = self.backbone_cls(cfg)
        self.lm_head = nn.Linear(cfg.hidden_size, cfg.vocab_size, bias=False)
        if cfg.tie_word_embeddings:
            self.lm_head.weight = self.model.embed_tokens.weight
        self.sp_group = None  # set by the trainer when Ulysses is on
        self.tp_group = None  # set by the tensor-parallel plan
        self.causal = True
        self.shift_labels = True
        self.loss_reduction = "mean"
        self.apply(self._init_weights)

    def _init_weights(self, m):
        std = self.config.initializer_range
        if isinstance(m, nn.Linear):
            nn.init.normal_(m.weight, mean=0.0, std=std)
            if m.bias is not None:
                nn.init.zeros_(m.bias)
        elif isinstance(m, nn.Embedding):
            nn.init.normal_(m.weight, mean=0.0, std=std)

    # -- helpers ---------------------------------------------------------------------------
    def gradient_checkpointing_enable(self, *_, **__):
        self.model.gradient_checkpointing = True

    def get_input_embeddings(self):
        return self.model.embed_tokens

    def num_parameters(self, exclude_embeddings: bool = False) -> int:
        seen, n = set(), 0
        for name, p in self.named_parameters():
            if id(p) in seen:
                continue
            seen.add(id(p))
            if exclude_embeddings and ("embed_tokens" in name):
                continue
            n += p.numel()
        return n

    def prepare_packed(self, input_ids, attention_mask=None, labels=None, position_ids=None, cu_seqlens=None):
        """Normalise the accepted input forms to a flat packed stream."""
        if input_ids is not None and input_ids.dim() == 2:
            if attention_mask is None:
                attention_mask = torch.ones_like(input_ids)
            ids, lab, pos, cu, idx = unpad_batch(input_ids, attention_mask, labels, position_ids)
            return ids, lab, pos, cu, idx
        T = input_ids.shape[0]
        if cu_seqlens is None:
            cu_seqlens = torch.tensor([0, T], dtype=torch.int32, device=input_ids.device)
        if position_ids is None:
            position_ids = positions_from_cu_seqlens(cu_seqlens, T)
        return input_ids, labels, position_ids, cu_seqlens.to(torch.int32), None

    def forward(
        self,
        input_ids: Optional[torch.Tensor] = None,
        attention_mask: Optional[torch.Tensor] = None,
        labels: Optional[torch.Tensor] = None,
        position_ids: Optional[torch.Tensor] = None,
        cu_seqlens: Optional[torch.Tensor] = None,
        max_seqlen: Optional[int] = None,
        inputs_embeds: Optional[torch.Tensor] = None,
        return_logits: bool = False,
        deepstack: Optional[List[torch.Tensor]] = None,
        deepstack_index: Optional[torch.Tensor] = None,
        kv_cache: Any = None,
        **unused,
    ) -> Dict[str, Any]:
        if kv_cache is not None and not self.supports_kv_cache:
            raise NotImplementedError(f"{type(self).__name__} has no key / value cache path")
        if inputs_embeds is None:
            ids, labels, pos, cu, _ = self.prepare_packed(input_ids, attention_mask, labels, position_ids, cu_seqlens)
        else:
            ids, pos, cu = None, position_ids, cu_seqlens.to(torch.int32)
        T_full = pos.shape[-1]
        if max_seqlen is None:
            max_seqlen = T_full  # an upper bound is enough: the kernels schedule from cu_seqlens
        if labels is None:
            shifted = None
        elif self.shift_labels:
            shifted = shift_labels_per_document(labels, cu)
        else:  # targets already aligned with their positions (masked-token objectives)
            shifted = labels
        cos, sin = self.model.rope_tables(pos)
        sp_group, tp_group = self.sp_group, self.tp_group
        sp_size, tp_size = sp.group_size(sp_group), sp.group_size(tp_group)
        if sp_size > 1 and tp_size > 1:
            raise NotImplementedError("Ulysses and tensor parallelism cannot be combined in one model")
        # sg: the group over which the token stream is split between blocks (Ulysses ranks, or
        # tensor-parallel ranks in the sequence-parallel regions)
        sg, sg_size = (tp_group, tp_size) if tp_size > 1 else (sp_group, sp_size)
        ctx = PackedContext(cu, int(max_seqlen), cos, sin, self.causal, sp_group, sp_size, tp_group, tp_size,
                            deepstack=deepstack, deepstack_index=deepstack_index)
        if kv_cache is not None:
            ctx.kv_cache = kv_cache  # positions of the new tokens come from ``kv_cache.advance`` through ``position_ids``
        if inputs_embeds is None:
            if sg_size > 1:
                ids = sp.slice_for_rank(sp.pad_to_multiple(ids, sg_size, 0), sg)
            inputs_embeds = self.model.embed_tokens(ids)
        elif sg_size > 1:
            inputs_embeds = sp.slice_for_rank(sp.pad_to_multiple(inputs_embeds, sg_size, 0), sg)
        if sg_size > 1:
            ctx.split_group, ctx.split_total = sg, T_full + (-T_full) % sg_size
            # padded tail tokens form a trailing pseudo-document
            pad = (-T_full) % sg_size
            if pad:
                ctx.cu_seqlens = torch.cat([cu, cu[-1:] + pad]).to(torch.int32)
                ctx.cos = sp.pad_to_multiple(cos, sg_size, 0)
                ctx.sin = sp.pad_to_multiple(sin, sg_size, 0)
            if shifted is not None:
                shifted = sp.slice_for_rank(sp.pad_to_multiple(shifted, sg_size, IGNORE_INDEX), sg)
        hidden = self.model(inputs_embeds, ctx)
        out: Dict[str, Any] = {"aux": ctx.aux}
        if return_logits:
            out["logits"] = F.linear(hidden, self.lm_head.weight)
        if shifted is not None:
            out["loss"] = self.compute_loss(hidden, shifted, sg, sg_size, averaged_by_fsdp=tp_size <= 1)
            n_valid = (shifted != IGNORE_INDEX).sum()
            out["num_tokens"] = n_valid
        out["hidden_states"] = hidden if labels is None else None
        return out

    def compute_loss(self, hidden, shifted, sp_group, sp_size, averaged_by_fsdp=True):
        w = _w(self.lm_head.weight)
        if sp_size > 1:
            # per-token losses on the local slice, then the SP-wide token-weighted mean;
            # the gather's backward scales by the group size because FSDP averages over
            # the flattened dp x cp mesh (see sequence_parallel.ulysses.gather_loss)
            per_tok = ce_ops.fused_linear_cross_entropy(hidden, w, shifted, "none")
            return sp.reduce_loss(per_tok, shifted != IGNORE_INDEX, sp_group, averaged_by_fsdp)
        return ce_ops.fused_linear_cross_entropy(hidden, w, shifted, self.loss_reduction)


def positions_from_cu_seqlens(cu_seqlens: torch.Tensor, total: int) -> torch.Tensor:
    """Per-document positions 0..len-1 for a packed stream (no host sync)."""
    starts = torch.zeros(total + 1, dtype=torch.long, device=cu_seqlens.device)
    inner = cu_seqlens[1:-1].long().clamp(max=total)
    lens = (cu_seqlens[1:-1] - cu_seqlens[:-2]).long()
    starts.index_add_(0, inner, lens)
    doc_start = torch.cumsum(starts[:total], 0)
    return torch.arange(total, device=cu_seqlens.device) - doc_start
