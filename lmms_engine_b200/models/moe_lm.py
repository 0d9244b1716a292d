"""Packed-varlen mixture-of-experts decoder (Qwen3-MoE family; shared-expert variant for
Qwen2-MoE / Qwen3.5-MoE style blocks).

Experts are stored fused, like ``transformers`` >= 5 does in memory:
``mlp.experts.gate_up_proj [E, 2I, H]`` and ``mlp.experts.down_proj [E, H, I]``; hub
checkpoints with per-expert ``mlp.experts.{i}.{gate,up,down}_proj.weight`` are converted on
load and emitted again on export, so merged checkpoints stay loadable upstream.

Replaces the patched HF forwards of src/lmms_engine/models/qwen3_moe/qwen3_moe_ops.py:130-322
and the aux-loss plumbing of src/lmms_engine/models/qwen3_moe/qwen3_moe_liger.py:27-167.
"""
from __future__ import annotations

import re
from dataclasses import dataclass, fields
from typing import Any, Dict, List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import gemm as gemm_ops
from ..ops import moe as moe_ops
from .decoder_lm import DecoderBackbone, DecoderConfig, DecoderLayer, DecoderLM, SwiGLUMLP


@dataclass
class MoEConfig(DecoderConfig):
    model_type: str = "qwen3_moe"
    num_experts: int = 128
    num_experts_per_tok: int = 8
    moe_intermediate_size: int = 768
    norm_topk_prob: bool = True
    router_aux_loss_coef: float = 1e-3
    output_router_logits: bool = True
    decoder_sparse_step: int = 1
    mlp_only_layers: Optional[List[int]] = None
    shared_expert_intermediate_size: int = 0

    def __post_init__(self):
        super().__post_init__()
        if self.mlp_only_layers is None:
            self.mlp_only_layers = []
        if self.architectures in (None, ["Qwen2ForCausalLM"], ["Qwen3ForCausalLM"]):
            self.architectures = ["Qwen3MoeForCausalLM"]

    def is_sparse_layer(self, i: int) -> bool:
        return i not in self.mlp_only_layers and self.num_experts > 0 and (i + 1) % self.decoder_sparse_step == 0


class _ScaleGrad(torch.autograd.Function):
    """Identity whose backward multiplies the gradient by ``factor``."""

    @staticmethod
    def forward(ctx, x, factor):
        ctx.factor = factor
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        return g * ctx.factor, None


class Experts(nn.Module):
    # set by the expert-parallel plan when the experts are NOT wrapped by a sharding wrapper (every expert lives on exactly
    # one rank): the dtype the grouped products run in (the parameters stay fp32 masters) and the factor that turns the
    # sum of the ranks' loss gradients, which the token exchange produces, into the gradient of their mean
    compute_dtype = None
    grad_scale = 1.0

    def __init__(self, n: int, hidden: int, inter: int):
        super().__init__()
        self.gate_up_proj = nn.Parameter(torch.empty(n, 2 * inter, hidden))
        self.down_proj = nn.Parameter(torch.empty(n, hidden, inter))
        self.num_experts, self.hidden, self.inter = n, hidden, inter

    def forward(self, xp: torch.Tensor, perm) -> torch.Tensor:
        """Grouped SwiGLU MLP over expert-major rows.  Every caller (the local path and the expert-parallel
        dispatchers) goes through ``forward`` so that a wrapper's hooks (FSDP2 unshard / mixed precision) run; under
        expert parallelism the stacked parameters are DTensors on the ep mesh and the rows are this rank's experts'."""
        gate_up, down = self.gate_up_proj, self.down_proj
        if hasattr(gate_up, "to_local"):
            gate_up, down = gate_up.to_local(), down.to_local()
        if self.grad_scale != 1.0 and torch.is_grad_enabled():
            gate_up, down = _ScaleGrad.apply(gate_up, self.grad_scale), _ScaleGrad.apply(down, self.grad_scale)
        if self.compute_dtype is not None and gate_up.dtype != self.compute_dtype:
            gate_up, down = gate_up.to(self.compute_dtype), down.to(self.compute_dtype)
        if xp.shape[0] > 0:
            return moe_ops.grouped_mlp(xp, gate_up, down, perm)
        # no rows for this rank's experts in this step: keep the parameters in the graph (their gradient hooks and
        # the collectives behind them must still run on every rank)
        return xp.new_zeros((0, self.hidden)) + 0.0 * (gate_up.sum() + down.sum()).to(xp.dtype)


class SparseMoeBlock(nn.Module):
    def __init__(self, cfg: MoEConfig):
        super().__init__()
        self.cfg = cfg
        self.gate = nn.Linear(cfg.hidden_size, cfg.num_experts, bias=False)
        self.experts = Experts(cfg.num_experts, cfg.hidden_size, cfg.moe_intermediate_size)
        if cfg.shared_expert_intermediate_size:
            self.shared_expert = SwiGLUMLP(cfg.hidden_size, cfg.shared_expert_intermediate_size)
            self.shared_expert_gate = nn.Linear(cfg.hidden_size, 1, bias=False)
        self.ep = None  # set by the expert-parallel plan: an ExpertParallel dispatcher

    def forward(self, x: torch.Tensor):
        cfg = self.cfg
        logits = gemm_ops.linear(x, self.gate.weight, None)
        probs, idx, w, counts = moe_ops.router_topk(logits, cfg.num_experts_per_tok, cfg.norm_topk_prob)
        if self.ep is not None:
            y = self.ep(x, idx, w, counts, self.experts)
        else:
            perm = moe_ops.build_permutation(idx, w, counts)
            xp = moe_ops.dispatch(x, perm)
            yp = self.experts(xp, perm)
            y = moe_ops.combine(yp, w, perm)
        if cfg.shared_expert_intermediate_size:
            s = self.shared_expert(x)
            y = y + torch.sigmoid(F.linear(x, self.shared_expert_gate.weight)) * s
        aux = moe_ops.load_balancing_loss(probs, counts, cfg.num_experts_per_tok)
        return y, aux


class MoEDecoderLayer(DecoderLayer):
    def build_mlp(self, cfg: MoEConfig, layer_idx: int):
        if cfg.is_sparse_layer(layer_idx):
            return SparseMoeBlock(cfg)
        return SwiGLUMLP(cfg.hidden_size, cfg.intermediate_size)


class MoEBackbone(DecoderBackbone):
    layer_cls = MoEDecoderLayer


_EXPERT_KEY = re.compile(r"^(.*\.mlp\.experts)\.(\d+)\.(gate_proj|up_proj|down_proj)\.weight$")


class MoEDecoderLM(DecoderLM):
    config_class = MoEConfig
    backbone_cls = MoEBackbone
    _no_split_modules = ["MoEDecoderLayer"]

    def _init_weights(self, m):
        super()._init_weights(m)
        if isinstance(m, Experts):
            nn.init.normal_(m.gate_up_proj, mean=0.0, std=self.config.initializer_range)
            nn.init.normal_(m.down_proj, mean=0.0, std=self.config.initializer_range)

    def forward(self, *args, **kwargs) -> Dict[str, Any]:
        out = super().forward(*args, **kwargs)
        aux = out.get("aux") or []
        if aux:
            aux_loss = torch.stack([a.float() for a in aux]).mean()
            out["aux_loss"] = aux_loss
            # per-token losses (``loss_reduction = "none"``, the log-probabilities of policy-gradient trainers) stay what they are
            if out.get("loss") is not None and out["loss"].dim() == 0 and self.config.router_aux_loss_coef:
                out["lm_loss"] = out["loss"].detach()
                out["loss"] = out["loss"] + self.config.router_aux_loss_coef * aux_loss.to(out["loss"].dtype)
        return out

    # ---- hub naming <-> fused experts --------------------------------------------------------
    @staticmethod
    def convert_hf_state_dict_static(sd: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        groups: Dict[str, Dict[int, Dict[str, torch.Tensor]]] = {}
        out: Dict[str, torch.Tensor] = {}
        for k, v in sd.items():
            m = _EXPERT_KEY.match(k)
            if m:
                groups.setdefault(m.group(1), {}).setdefault(int(m.group(2)), {})[m.group(3)] = v
            else:
                out[k] = v
        for prefix, experts in groups.items():
            ids = sorted(experts)
            out[prefix + ".gate_up_proj"] = torch.stack(
                [torch.cat([experts[i]["gate_proj"], experts[i]["up_proj"]], 0) for i in ids], 0)
            out[prefix + ".down_proj"] = torch.stack([experts[i]["down_proj"] for i in ids], 0)
        return out

    def convert_hf_state_dict(self, sd):
        return self.convert_hf_state_dict_static(sd)

    @staticmethod
    def export_hf_state_dict_static(sd: Dict[str, torch.Tensor], config=None) -> Dict[str, torch.Tensor]:
        out: Dict[str, torch.Tensor] = {}
        for k, v in sd.items():
            if k.endswith(".mlp.experts.gate_up_proj"):
                prefix = k[: -len(".gate_up_proj")]
                inter = v.shape[1] // 2
                for e in range(v.shape[0]):
                    out[f"{prefix}.{e}.gate_proj.weight"] = v[e, :inter].contiguous()
                    out[f"{prefix}.{e}.up_proj.weight"] = v[e, inter:].contiguous()
            elif k.endswith(".mlp.experts.down_proj"):
                prefix = k[: -len(".down_proj")]
                for e in range(v.shape[0]):
                    out[f"{prefix}.{e}.down_proj.weight"] = v[e].contiguous()
            else:
                out[k] = v
        return out

    def export_hf_state_dict(self, sd):
        return self.export_hf_state_dict_static(sd, None)
