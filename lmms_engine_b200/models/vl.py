"""Vision-language models: a vision tower feeding a packed decoder through placeholder
tokens, with multimodal rotary positions (Qwen2.5-VL: sectioned; Qwen3-VL: interleaved, plus
deepstack features added to the first decoder layers).

Replaces the patched HF forwards of src/lmms_engine/models/qwen2_5_vl/qwen2_5_vl_ops.py:72-234
and src/lmms_engine/models/qwen3_vl/qwen3_vl_ops.py:47-142, 284-442.  Parameter names of the
upstream checkpoints (``model.visual.*``, ``model.language_model.*``, ``lm_head.*``) are
mapped in ``convert_hf_state_dict`` / ``export_hf_state_dict``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

import torch
import torch.nn as nn

from ..ops import index as index_ops
from . import mrope
from .decoder_lm import DecoderConfig, DecoderLM
from .moe_lm import MoEConfig, MoEDecoderLM
from .vision import Qwen25VisionTower, Qwen3VisionTower, VisionConfig


@dataclass
class VLConfig:
    model_type: str = "qwen2_5_vl"
    text_config: Any = None
    vision_config: Any = None
    image_token_id: int = 151655
    video_token_id: int = 151656
    vision_start_token_id: int = 151652
    vision_end_token_id: int = 151653
    tie_word_embeddings: bool = False
    architectures: Optional[List[str]] = None
    extra: Dict[str, Any] = field(default_factory=dict)

    @property
    def is_qwen3(self) -> bool:
        return self.model_type.startswith("qwen3")

    @property
    def is_rice(self) -> bool:
        """LLaVA-OneVision-1.5: Rice tower, Qwen3 decoder, plain 1-D rotary positions."""
        return self.model_type.startswith("llavaonevision1_5")

    @property
    def is_ov2(self) -> bool:
        """LLaVA-OneVision-2: position-carrying patch tower, Qwen3 decoder, plain 1-D rotary positions."""
        return self.model_type.startswith("llava_onevision2")

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "VLConfig":
        d = dict(d)
        mt = d.get("model_type", "qwen2_5_vl")
        text = dict(d.pop("text_config", None) or {})
        vis = dict(d.pop("vision_config", None) or {})
        # older Qwen2.5-VL configs keep the text fields at the top level
        if not text:
            text = {k: v for k, v in d.items() if k in {f for f in DecoderConfig.__dataclass_fields__}}
        moe = "moe" in mt
        rice = mt.startswith("llavaonevision1_5") or mt.startswith("llava_onevision2")
        if mt.startswith("llava_onevision2"):
            text["model_type"] = "qwen3"
            text["mrope_section"] = None
            vis["model_type"] = "onevision2_vit"
            vis.setdefault("temporal_patch_size", 1)
            vis.setdefault("hidden_act", "gelu")
            vis.setdefault("hidden_size", 1024)
            vis.setdefault("intermediate_size", 4096)
            vis.setdefault("depth", 24)
        elif rice:
            text["model_type"] = "qwen3"  # q/k RMSNorm on the head dimension, no attention bias
            text["mrope_section"] = None
            vis["model_type"] = "rice_vit"
            vis.setdefault("temporal_patch_size", 1)
            vis.setdefault("hidden_act", "gelu")
            vis.setdefault("hidden_size", 1024)
            vis.setdefault("intermediate_size", 4096)
            vis.setdefault("depth", 24)
            if "text_hidden_size" in vis:
                vis.setdefault("out_hidden_size", vis["text_hidden_size"])
        text["model_type"] = text.get("model_type") or ("qwen3_moe" if moe else ("qwen3" if mt.startswith("qwen3") else "qwen2"))
        if text["model_type"].endswith("_text"):
            text["model_type"] = "qwen3_moe" if moe else ("qwen3" if mt.startswith("qwen3") else "qwen2")
        for key in ("rope_parameters", "rope_scaling"):  # hub configs keep the sections inside the rope dict
            sect = (text.get(key) or {}).get("mrope_section") if isinstance(text.get(key), dict) else None
            if sect and "mrope_section" not in text:
                text["mrope_section"] = list(sect)
        if rice:
            pass
        elif mt.startswith("qwen3"):
            text.setdefault("mrope_mode", "interleaved")
            text.setdefault("mrope_section", [24, 20, 20])
        else:
            text.setdefault("mrope_mode", "sectioned")
            text.setdefault("mrope_section", [16, 24, 24])
        vis.setdefault("model_type", mt)
        if mt.startswith("qwen3"):
            vis.setdefault("hidden_act", "gelu_pytorch_tanh")
            vis.setdefault("patch_size", 16)
            vis.setdefault("depth", 27)
            vis.setdefault("hidden_size", 1152)
            vis.setdefault("intermediate_size", 4304)
        if mt.startswith("qwen3_5"):
            # hybrid Gated-DeltaNet decoder; its vision tower is the Qwen3-VL one without deepstack taps
            from .qwen3_5 import Qwen35Config, Qwen35MoEConfig

            text["model_type"] = "qwen3_5_moe_text" if moe else "qwen3_5_text"
            vis.setdefault("deepstack_visual_indexes", [])
            tcfg = (Qwen35MoEConfig if moe else Qwen35Config).from_dict(text)
        else:
            tcfg = (MoEConfig if moe else DecoderConfig).from_dict(text)
        vis.setdefault("out_hidden_size", tcfg.hidden_size)
        vcfg = VisionConfig.from_dict(vis)
        known = {"image_token_id", "video_token_id", "vision_start_token_id", "vision_end_token_id", "tie_word_embeddings", "architectures"}
        kw = {k: d[k] for k in known if k in d}
        extra = {k: v for k, v in d.items() if k not in known and k != "model_type" and k not in DecoderConfig.__dataclass_fields__}
        return cls(model_type=mt, text_config=tcfg, vision_config=vcfg, extra=extra, **kw)

    def to_dict(self) -> Dict[str, Any]:
        d = {"model_type": self.model_type, "text_config": self.text_config.to_dict(), "vision_config": self.vision_config.to_dict(),
             "image_token_id": self.image_token_id, "video_token_id": self.video_token_id,
             "vision_start_token_id": self.vision_start_token_id, "vision_end_token_id": self.vision_end_token_id,
             "tie_word_embeddings": self.tie_word_embeddings,
             "architectures": self.architectures or [
                 "LlavaOnevision2ForConditionalGeneration" if self.is_ov2 else
                 "LLaVAOneVision1_5_ForConditionalGeneration" if self.is_rice else
                 "Qwen3VLForConditionalGeneration" if self.is_qwen3 else "Qwen2_5_VLForConditionalGeneration"]}
        d.update(self.extra)
        return d

    # the FLOPs counter and the trainer look at text fields through the top-level config
    def __getattr__(self, name):
        if name in ("text_config", "vision_config") or name.startswith("__"):
            raise AttributeError(name)
        return getattr(self.text_config, name)


class VLModel(nn.Module):
    """``visual`` tower + ``language_model`` decoder."""

    config_class = VLConfig
    _no_split_modules = ["DecoderLayer", "MoEDecoderLayer", "VisionBlock", "RiceBlock"]

    def __init__(self, cfg: VLConfig):
        super().__init__()
        self.config = cfg
        if cfg.is_ov2:
            from .llava_ov2 import OneVisionTower

            self.visual = OneVisionTower(cfg.vision_config)
        elif cfg.is_rice:
            from .rice import RiceVisionTower

            self.visual = RiceVisionTower(cfg.vision_config)
        else:
            self.visual = (Qwen3VisionTower if cfg.is_qwen3 else Qwen25VisionTower)(cfg.vision_config)
        self.language_model = self._decoder_class(cfg.text_config)(cfg.text_config)

    @staticmethod
    def _decoder_class(text_config):
        from .qwen3_5 import Qwen35Config, Qwen35LM, Qwen35MoEConfig, Qwen35MoELM

        if isinstance(text_config, Qwen35MoEConfig):
            return Qwen35MoELM
        if isinstance(text_config, Qwen35Config):
            return Qwen35LM
        return MoEDecoderLM if isinstance(text_config, MoEConfig) else DecoderLM

    # ViT frame balancing over the flattened dp x cp ranks (set by the trainer / monkey_patch_kwargs)
    vit_frame_parallel = False
    vit_group = None
    # under sequence parallelism every rank of a group runs the tower on its share of the sample's frames
    sp_split_vit = True

    # the trainer toggles these on whatever model it gets
    @property
    def sp_group(self):
        return self.language_model.sp_group

    @sp_group.setter
    def sp_group(self, g):
        self.language_model.sp_group = g

    def gradient_checkpointing_enable(self, *a, **k):
        self.language_model.gradient_checkpointing_enable()
        self.visual.gradient_checkpointing = True

    def get_input_embeddings(self):
        return self.language_model.model.embed_tokens

    def embed_multimodal(self, ids, pixel_values, image_grid_thw, pixel_values_videos, video_grid_thw, embed_ids=None):
        """Token embeddings with image / video features written over their placeholders (``embed_ids``: a parallel
        stream whose tokens are embedded instead, placeholders still found in ``ids``)."""
        cfg = self.config
        emb = self.language_model.model.embed_tokens(ids if embed_ids is None else embed_ids)
        deep_all, index_all = None, None
        for pix, grid, tok in ((pixel_values, image_grid_thw, cfg.image_token_id),
                               (pixel_values_videos, video_grid_thw, cfg.video_token_id)):
            balanced = self.vit_frame_parallel and self.vit_group is not None
            if (pix is None or pix.numel() == 0) and not balanced:
                continue
            from ..parallel.sequence_parallel import ulysses as sp_mod

            sp_n = sp_mod.group_size(self.language_model.sp_group)
            split_sp = sp_n > 1 and self.sp_split_vit and not (cfg.is_rice or cfg.is_ov2)
            if balanced:
                # every rank takes part in the exchange, also one whose batch has no frames of this kind
                from ..parallel.vit_parallel import balanced_vit_forward

                vc = cfg.vision_config
                if pix is None:
                    pix = emb.new_zeros((0, vc.in_channels * vc.temporal_patch_size * vc.patch_size ** 2))
                    grid = torch.zeros((0, 3), dtype=torch.long, device=emb.device)
                run = lambda p_, g_: balanced_vit_forward(self.visual, p_, g_, self.vit_group)  # noqa: E731
            else:
                run = self.visual
            if split_sp:
                # the ranks of a sequence-parallel group hold the same sample: each runs the tower on its share of the
                # frames (and only that share enters the balancing), the features are gathered back
                from ..parallel.vit_parallel.frame_parallel import sp_sharded_vit_forward

                out = sp_sharded_vit_forward(self.visual, pix.to(emb.dtype), grid, self.language_model.sp_group, run, always_run=balanced)
            else:
                out = run(pix.to(emb.dtype), grid)
            if pix.shape[0] == 0:
                continue
            feats, deep = out if isinstance(out, tuple) else (out, None)
            mask = ids == tok
            # the k-th placeholder takes the k-th feature row: prefix count, no host round trip
            src = (torch.cumsum(mask, 0) - 1).clamp(min=0)
            gathered = feats.index_select(0, src.clamp(max=feats.shape[0] - 1)).to(emb.dtype)
            emb = torch.where(mask.unsqueeze(-1), gathered, emb)
            if deep:
                pos = torch.nonzero(mask, as_tuple=False).flatten()
                if deep_all is None:
                    deep_all, index_all = [d_ for d_ in deep], pos
                else:
                    deep_all = [torch.cat([a, b], 0) for a, b in zip(deep_all, deep)]
                    index_all = torch.cat([index_all, pos])
        return emb, deep_all, index_all

    def forward(self, input_ids=None, attention_mask=None, labels=None, position_ids=None, cu_seqlens=None,
                pixel_values=None, image_grid_thw=None, pixel_values_videos=None, video_grid_thw=None,
                second_per_grid_ts=None, **kw):
        cfg = self.config
        lm = self.language_model
        had_mrope = position_ids is not None and position_ids.dim() >= 2 and position_ids.shape[-2] == 3
        # a generation step (key / value cache present) states the positions of its new tokens, whatever their form;
        # otherwise one-dimensional positions are the collator's per-document counters, which images and videos replace
        had_mrope = had_mrope or (position_ids is not None and kw.get("kv_cache") is not None)
        ids, labels, pos, cu, _ = lm.prepare_packed(input_ids, attention_mask, labels, position_ids if had_mrope else None, cu_seqlens)
        if not had_mrope and not cfg.is_rice and not cfg.is_ov2:
            grids, secs = [], []
            for g, is_video in ((image_grid_thw, False), (video_grid_thw, True)):
                if g is None:
                    continue
                gl = g.tolist() if torch.is_tensor(g) else list(g)
                grids += gl
                if is_video and second_per_grid_ts is not None and not cfg.is_qwen3:
                    secs += list(second_per_grid_ts.tolist() if torch.is_tensor(second_per_grid_ts) else second_per_grid_ts)
                else:
                    secs += [0.0] * len(gl)
            if grids:
                # NOTE: grids are consumed in stream order; streams that interleave images and
                # videos should ship precomputed positions from the processor
                pos = mrope.build_mrope_positions(
                    ids, cu, (cfg.image_token_id, cfg.video_token_id), grids, secs, cfg.vision_config.spatial_merge_size,
                    cfg.vision_config.tokens_per_second if not cfg.is_qwen3 else 0.0).to(ids.device)
        emb, deep, deep_idx = self.embed_multimodal(ids, pixel_values, image_grid_thw, pixel_values_videos, video_grid_thw)
        return lm(inputs_embeds=emb, labels=labels, position_ids=pos, cu_seqlens=cu, deepstack=deep, deepstack_index=deep_idx, **kw)

    # ---- hub names ----------------------------------------------------------------------------
    def convert_hf_state_dict(self, sd):
        out = {}
        for k, v in sd.items():
            if k.startswith("model.visual."):
                out["visual." + k[len("model.visual."):]] = v
            elif k.startswith("visual."):
                out[k] = v
            elif k.startswith("model.language_model."):
                out["language_model.model." + k[len("model.language_model."):]] = v
            elif k.startswith("lm_head."):
                out["language_model." + k] = v
            elif k.startswith("model."):
                out["language_model." + k] = v
            else:
                out[k] = v
        if hasattr(self.language_model, "convert_hf_state_dict"):
            out = self.language_model.convert_hf_state_dict(out)
        return out

    @staticmethod
    def export_hf_state_dict_static(sd, config=None):
        out = {}
        for k, v in sd.items():
            if k.startswith("visual."):
                out["model." + k] = v
            elif k.startswith("language_model.model."):
                out["model.language_model." + k[len("language_model.model."):]] = v
            elif k.startswith("language_model.lm_head."):
                out[k[len("language_model."):]] = v
            else:
                out[k] = v
        return MoEDecoderLM.export_hf_state_dict_static(out, config)

    def export_hf_state_dict(self, sd):
        return self.export_hf_state_dict_static(sd, None)
