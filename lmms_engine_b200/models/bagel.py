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
from typing import Any, Dict, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import cross_entropy as ce_ops
from .decoder_lm import (IGNORE_INDEX, DecoderBackbone, DecoderConfig, DecoderLayer, DecoderLM, PackedContext, RMSNorm,
                         SwiGLUMLP, _w, shift_labels_per_document)
from .diffusion import timestep_embedding


@dataclass
class BagelConfig(DecoderConfig):
    model_type: str = "bagel"
    latent_channels: int = 16
    latent_patch_size: int = 2
    max_latent_size: int = 64
    timestep_shift: float = 1.0
    ce_weight: float = 1.0
    mse_weight: float = 1.0
    use_mot: bool = True


class MoTLayer(DecoderLayer):
    """Decoder layer whose norm + MLP exist twice: one set for understanding (text / ViT) tokens,
    one for generation (latent) tokens; attention projections are shared."""

    def __init__(self, cfg: BagelConfig, layer_idx: int):
        super().__init__(cfg, layer_idx)
        if cfg.use_mot:
            self.mlp_moe_gen = SwiGLUMLP(cfg.hidden_size, cfg.intermediate_size)
            self.post_attention_layernorm_moe_gen = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps)

    def forward(self, h, residual, ctx: PackedContext):
        if residual is None:
            residual = h
            x = self.input_layernorm(h)
        else:
            x, residual = self.input_layernorm(h, residual)
        a = self.self_attn(x, ctx)
        gen = getattr(ctx, "gen_index", None)
        if gen is None or not hasattr(self, "mlp_moe_gen"):
            x, residual = self.post_attention_layernorm(a, residual)
            return self.mlp(x), residual
        residual = residual + a
        und = ctx.und_index
        out = torch.zeros_like(residual)
        if und.numel():
            out = out.index_copy(0, und, self.mlp(self.post_attention_layernorm(residual.index_select(0, und))))
        if gen.numel():
            out = out.index_copy(0, gen, self.mlp_moe_gen(self.post_attention_layernorm_moe_gen(residual.index_select(0, gen))))
        return out, residual


class BagelBackbone(DecoderBackbone):
    layer_cls = MoTLayer


class Bagel(DecoderLM):
    config_class = BagelConfig
    backbone_cls = BagelBackbone
    _no_split_modules = ["MoTLayer"]

    def __init__(self, cfg: BagelConfig):
        super().__init__(cfg)
        pd = cfg.latent_channels * cfg.latent_patch_size ** 2
        self.vae2llm = nn.Linear(pd, cfg.hidden_size)
        self.llm2vae = nn.Linear(cfg.hidden_size, pd)
        self.time_embedder = nn.Sequential(nn.Linear(256, cfg.hidden_size), nn.SiLU(), nn.Linear(cfg.hidden_size, cfg.hidden_size))
        self.latent_pos_embed = nn.Embedding(cfg.max_latent_size ** 2, cfg.hidden_size)

    def forward(self, input_ids=None, labels=None, cu_seqlens=None, position_ids=None, latent_tokens=None,
                latent_index=None, latent_pos=None, timesteps=None, latent_loss_mask=None, **kw) -> Dict[str, Any]:
        """Packed stream of length T.  ``latent_tokens [G, C*p*p]`` are clean VAE patches that sit at
        stream positions ``latent_index [G]`` (their ``input_ids`` entries are ignored);
        ``timesteps [G]`` in (0,1) give each patch's noise level (same value within an image)."""
        cfg = self.config
        ids, labels, pos, cu, _ = self.prepare_packed(input_ids, None, labels, position_ids, cu_seqlens)
        emb = self.model.embed_tokens(ids)
        out: Dict[str, Any] = {}
        G = 0 if latent_tokens is None else latent_tokens.shape[0]
        noise = target = None
        if G:
            t = timesteps.float()
            t = cfg.timestep_shift * t / (1 + (cfg.timestep_shift - 1) * t)
            noise = torch.randn_like(latent_tokens.float())
            x_t = (1 - t[:, None]) * latent_tokens.float() + t[:, None] * noise
            target = noise - latent_tokens.float()
            g = self.vae2llm(x_t.to(emb.dtype)) + self.time_embedder(timestep_embedding(t * 1000, 256).to(emb.dtype))
            g = g + self.latent_pos_embed(latent_pos)
            emb = emb.index_copy(0, latent_index, g.to(emb.dtype))
        cos, sin = self.model.rope_tables(pos)
        ctx = PackedContext(cu, int(pos.shape[-1]), cos, sin, True)
        if G:
            mask = torch.zeros(ids.shape[0], dtype=torch.bool, device=ids.device)
            mask[latent_index] = True
            ctx.gen_index = latent_index
            ctx.und_index = torch.nonzero(~mask, as_tuple=False).flatten()
        hidden = self.model(emb, ctx)
        ce = mse = None
        if labels is not None:
            shifted = shift_labels_per_document(labels, cu)
            ce = ce_ops.fused_linear_cross_entropy(hidden, _w(self.lm_head.weight), shifted, "mean")
        if G:
            pred = self.llm2vae(hidden.index_select(0, latent_index)).float()
            err = ((pred - target) ** 2).mean(-1)
            if latent_loss_mask is not None:  # clean condition images carry no loss
                keep = latent_loss_mask.to(err.dtype)
                mse = (err * keep).sum() / keep.sum().clamp(min=1.0)
            else:
                mse = err.mean()
            out["velocity"] = pred
        loss = 0.0
        if ce is not None:
            loss = loss + cfg.ce_weight * ce
        if mse is not None:
            loss = loss + cfg.mse_weight * mse
        out.update(loss=loss, ce=ce.detach() if ce is not None else None, mse=mse.detach() if mse is not None else None)
        return out

    # ---- flow-GRPO -----------------------------------------------------------------------------
    @staticmethod
    def sde_step_with_logprob(v, x, t, dt, noise_level: float = 0.7, prev_sample=None, generator=None):
        """One reverse-time SDE step of the rectified flow (t: 1 = noise -> 0 = data) together with
        the Gaussian log-probability of the sample it produced, averaged over dimensions."""
        t = t.view(-1, *([1] * (x.dim() - 1)))
        std = noise_level * torch.sqrt(t / (1 - torch.where(t == 1, torch.full_like(t, 1 - 1e-3), t)).clamp(min=1e-3))
        mean = x * (1 + std ** 2 / (2 * t) * dt) + v * (1 + std ** 2 * (1 - t) / (2 * t)) * dt
        sd = std * math.sqrt(abs(dt))
        if prev_sample is None:
            prev_sample = mean + sd * torch.randn(x.shape, device=x.device, generator=generator)
        logp = (-((prev_sample.detach() - mean) ** 2) / (2 * sd ** 2) - torch.log(sd) - 0.5 * math.log(2 * math.pi))
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
