"""Assemble the initial checkpoint of a composite model from the checkpoints of its parts.

    python -m lmms_engine_b200.tools.prepare_init_weight --model-type aero --config aero_config.json \\
        --part language_model=Qwen2.5-7B-Instruct --part audio_tower=Qwen2-Audio-7B/audio_tower \\
        --add-tokens 3 --pad-vocab-to 64 --output ./aero_init

Every ``--part PREFIX=DIR`` loads a safetensors / ``pytorch_model.bin`` directory and places its tensors under
``PREFIX`` of the new model (the part's own ``model.`` / hub prefixes are tried as they are and with the common
wrappers stripped); parameters that no part covers keep the model's initialisation (projectors, merger).  When the
vocabulary grows, the new embedding and output rows are drawn from a Gaussian fitted to the existing rows with the
covariance scaled by 1e-5, so new tokens start near the mean embedding.

The reference spreads this over per-family scripts (tools/prepare_init_weight/prepare_aero.py:44-133,
prepare_aero_omni.py, prepare_aero_realtime.py:164-342, prepare_rae_siglip2.py:84-202).  Here the composer is generic
and the families are RECIPES that turn a few checkpoint directories into (model type, configuration, parts, new tokens):

    python -m lmms_engine_b200.tools.prepare_init_weight --recipe aero --language-model Qwen2.5-7B-Instruct \
        --audio-model Qwen2-Audio-7B-Instruct --output ./aero_init
    python -m lmms_engine_b200.tools.prepare_init_weight --recipe aero_realtime --vision-model Qwen3-VL-8B-Instruct \
        --audio-model Qwen2-Audio-7B-Instruct --output ./aero_rt_init [--skip-weights]
    python -m lmms_engine_b200.tools.prepare_init_weight --recipe rae_siglip2 --vision-model siglip2-base-patch16-256 \
        --output ./rae_init [--latent-stats stats.pt]

A recipe also extends and saves the tokenizer (when the language model's directory holds one that ``transformers`` can
load) and writes the token ids it assigned into the configuration.
"""
from __future__ import annotations

import argparse
import json
import os
from typing import Dict, List, Optional, Tuple

import torch

from ..mapping_func import create_model_from_config
from ..models import hf_io

_STRIP = ("", "model.", "thinker.", "language_model.", "model.language_model.", "audio_tower.", "thinker.audio_tower.",
          "visual.", "model.visual.", "vision_model.", "vision_tower.vision_model.", "vision_tower.")


def place_part(own: Dict[str, torch.Tensor], prefix: str, part: Dict[str, torch.Tensor]) -> Tuple[Dict[str, torch.Tensor], List[str]]:
    """Tensors of ``part`` that fit a parameter under ``prefix`` (same shape), and the part keys left over."""
    wanted = {k[len(prefix) + 1:]: k for k in own if k.startswith(prefix + ".")}
    best: Dict[str, torch.Tensor] = {}
    for strip in _STRIP:
        hit = {}
        for k, v in part.items():
            if not k.startswith(strip):
                continue
            name = k[len(strip):]
            if name in wanted and tuple(own[wanted[name]].shape) == tuple(v.shape):
                hit[wanted[name]] = v
        if len(hit) > len(best):
            best = hit
    used = {id(v) for v in best.values()}
    return best, [k for k, v in part.items() if id(v) not in used]


def grow_vocab(rows: torch.Tensor, new_rows: int, generator=None) -> torch.Tensor:
    """``rows [V, H]`` -> ``[V + new_rows, H]`` with the added rows sampled around the mean row."""
    if new_rows <= 0:
        return rows
    x = rows.float()
    mu = x.mean(0)
    centred = x - mu
    sigma = centred.T @ centred / x.shape[0]
    # sample through the Cholesky factor of the scaled covariance (jitter keeps it positive definite)
    L = torch.linalg.cholesky(1e-5 * sigma + 1e-10 * torch.eye(x.shape[1]))
    z = torch.randn(new_rows, x.shape[1], generator=generator)
    return torch.cat([rows, (mu + z @ L.T).to(rows.dtype)], 0)


def assemble(model_type: str, config: dict, parts: Dict[str, str], add_tokens: int = 0, pad_vocab_to: int = 1,
             dtype: torch.dtype = torch.bfloat16, seed: int = 0):
    torch.manual_seed(seed)
    gen = torch.Generator().manual_seed(seed)
    text = config.get("text_config", config)
    old_vocab = int(text["vocab_size"])
    new_vocab = old_vocab + add_tokens
    new_vocab = (new_vocab + pad_vocab_to - 1) // pad_vocab_to * pad_vocab_to
    text["vocab_size"] = new_vocab
    model = create_model_from_config(model_type, config)
    own = model.state_dict()
    report = {}
    for prefix, path in parts.items():
        part = hf_io.read_state_dict(path)
        # a part saved with the old vocabulary: grow its embedding rows before matching shapes
        if new_vocab != old_vocab:
            for k in list(part):
                if part[k].dim() == 2 and part[k].shape[0] == old_vocab and ("embed_tokens" in k or "lm_head" in k):
                    part[k] = grow_vocab(part[k], new_vocab - old_vocab, gen)
        placed, left = place_part(own, prefix, part)
        if not placed:
            raise KeyError(f"no tensor of {path} fits a parameter under '{prefix}.'")
        for k, v in placed.items():
            own[k].copy_(v.to(own[k].dtype))
        report[prefix] = {"placed": len(placed), "unused": len(left)}
    covered = sum(r["placed"] for r in report.values())
    report["fresh"] = len(own) - covered
    return model.to(dtype), report


# ---- family recipes ---------------------------------------------------------------------------------------------
def _read_config(path: str) -> dict:
    with open(os.path.join(path, "config.json")) as f:
        return json.load(f)


def _extend_tokenizer(path: str, tokens: List[str], output: Optional[str]):
    """Token ids of ``tokens`` after adding the missing ones to the tokenizer in ``path``; without a loadable
    tokenizer the ids continue the configured vocabulary."""
    if not any(os.path.exists(os.path.join(path, f)) for f in ("tokenizer.json", "tokenizer_config.json", "vocab.json", "tokenizer.model")):
        return None
    try:
        from transformers import AddedToken, AutoTokenizer

        tok = AutoTokenizer.from_pretrained(path, use_fast=True)
    except Exception:  # noqa: BLE001 - no tokenizer files, or a tokenizer class that is not installed
        return None
    for t in tokens:
        if t not in tok.get_vocab():
            tok.add_tokens(AddedToken(t, special=True, normalized=False), special_tokens=True)
    if output:
        tok.save_pretrained(output)
    return {t: tok.convert_tokens_to_ids(t) for t in tokens}, len(tok)


def _assign_ids(lm_dir: str, text_cfg: dict, tokens: List[str], output: Optional[str]):
    got = _extend_tokenizer(lm_dir, tokens, output)
    if got is not None:
        ids, size = got
        return ids, max(0, size - int(text_cfg["vocab_size"]))
    base = int(text_cfg["vocab_size"])
    return {t: base + i for i, t in enumerate(tokens)}, len(tokens)


def recipe_aero(a):
    """Language model + Whisper-style audio tower (Qwen2-Audio's, or the thinker's tower of a Qwen2.5-Omni checkpoint with
    ``--recipe aero_omni``) + a fresh linear projector; three new tokens ``<image> <video> <|AUDIO|>``."""
    text = _read_config(a.language_model)
    src = _read_config(a.audio_model)
    audio = (src.get("thinker_config", {}).get("audio_config") if a.recipe == "aero_omni" else src.get("audio_config")) or {}
    ids, added = _assign_ids(a.language_model, text, ["<image>", "<video>", "<|AUDIO|>"], a.output)
    cfg = {"model_type": "aero", "text_config": text, "audio_config": audio, "audio_token_index": ids["<|AUDIO|>"]}
    if a.recipe == "aero_omni":
        cfg["audio_config"] = dict(audio, model_type="qwen2_5_omni_audio_encoder")
    return "aero", cfg, {"language_model": a.language_model, "audio_tower": a.audio_model}, added


REALTIME_TOKENS = ["<|audio_start|>", "<|audio_end|>", "<|audio_pad|>", "<|rt_start|>", "<|rt_pad|>", "<|rt_speak|>", "<|rt_end|>"]


def recipe_aero_realtime(a):
    """Vision-language backbone (qwen3_vl / qwen3_vl_moe / qwen3_5 / qwen3_5_moe) + streaming audio encoder + fresh
    projector; the audio and realtime control tokens are added to the backbone's tokenizer."""
    vl = _read_config(a.vision_model)
    text = dict(vl.get("text_config") or {})
    text["tie_word_embeddings"] = vl.get("tie_word_embeddings", False)
    audio = dict(hidden_size=a.audio_hidden_size, intermediate_size=a.audio_intermediate_size, num_hidden_layers=a.audio_layers,
                 num_attention_heads=a.audio_heads, head_dim=a.audio_hidden_size // a.audio_heads, num_mel_bins=128,
                 sliding_window=a.audio_sliding_window, conv_padding=a.audio_padding_mode)
    ids, added = _assign_ids(a.vision_model, text, REALTIME_TOKENS, a.output)
    cfg = {"model_type": "aero_realtime", "backbone_family": a.backbone_family, "text_config": text, "vision_config": vl.get("vision_config"),
           "audio_config": audio, "downsample_factor": a.downsample_factor,
           "image_token_index": vl.get("image_token_id"), "video_token_index": vl.get("video_token_id"),
           "vision_start_token_index": vl.get("vision_start_token_id"), "audio_token_index": ids["<|audio_pad|>"],
           "audio_start_token_index": ids["<|audio_start|>"], "audio_end_token_index": ids["<|audio_end|>"],
           "rt_start_token_index": ids["<|rt_start|>"], "rt_pad_token_index": ids["<|rt_pad|>"],
           "rt_speak_token_index": ids["<|rt_speak|>"], "rt_end_token_index": ids["<|rt_end|>"]}
    parts = {"language_model": a.vision_model, "visual": a.vision_model}
    if a.audio_model:
        parts["audio_tower"] = a.audio_model
    return "aero_realtime", cfg, parts, added


def recipe_rae_siglip2(a):
    """SigLIP(2) vision encoder (frozen) + a fresh MAE-style decoder of the ViT-XL size, optional latent statistics."""
    src = _read_config(a.vision_model)
    enc = dict(src.get("vision_config") or src)
    if a.encoder_input_size:
        enc["image_size"] = int(a.encoder_input_size)
    dec = dict(decoder_hidden_size=1152, decoder_num_hidden_layers=28, decoder_num_attention_heads=16, decoder_intermediate_size=4096)
    if a.decoder_config:
        with open(a.decoder_config) as f:
            dec.update(json.load(f))
    cfg = {"model_type": "rae_siglip", "encoder_config": enc, "decoder_config": dec, "noise_tau": a.noise_tau, "eps": a.eps,
           "reshape_to_2d": not a.no_reshape_to_2d}
    if a.latent_stats:
        stats = torch.load(a.latent_stats, map_location="cpu")
        cfg["latent_mean"], cfg["latent_var"] = stats["mean"].float().tolist(), stats["var"].float().tolist()
    parts = {"encoder": a.vision_model}
    if a.decoder_checkpoint:
        parts["decoder"] = a.decoder_checkpoint
    return "rae_siglip", cfg, parts, 0


RECIPES = {"aero": recipe_aero, "aero_omni": recipe_aero, "aero_realtime": recipe_aero_realtime, "rae_siglip2": recipe_rae_siglip2}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--recipe", choices=sorted(RECIPES), default=None, help="a family recipe instead of --model-type / --config / --part")
    ap.add_argument("--language-model", default=None)
    ap.add_argument("--vision-model", default=None)
    ap.add_argument("--audio-model", default=None)
    ap.add_argument("--backbone-family", default="qwen3_vl")
    ap.add_argument("--downsample-factor", type=int, default=4)
    ap.add_argument("--audio-hidden-size", type=int, default=1280)
    ap.add_argument("--audio-intermediate-size", type=int, default=5120)
    ap.add_argument("--audio-layers", type=int, default=32)
    ap.add_argument("--audio-heads", type=int, default=20)
    ap.add_argument("--audio-sliding-window", type=int, default=750)
    ap.add_argument("--audio-padding-mode", default="causal")
    ap.add_argument("--decoder-config", default=None)
    ap.add_argument("--decoder-checkpoint", default=None)
    ap.add_argument("--latent-stats", default=None)
    ap.add_argument("--encoder-input-size", type=int, default=None)
    ap.add_argument("--noise-tau", type=float, default=0.8)
    ap.add_argument("--eps", type=float, default=1e-5)
    ap.add_argument("--no-reshape-to-2d", action="store_true")
    ap.add_argument("--skip-weights", action="store_true", help="write configuration (and tokenizer) only")
    ap.add_argument("--model-type", default=None)
    ap.add_argument("--config", default=None, help="json file with the composite model's configuration")
    ap.add_argument("--part", action="append", default=[], help="PREFIX=DIR, repeatable")
    ap.add_argument("--add-tokens", type=int, default=0)
    ap.add_argument("--pad-vocab-to", type=int, default=1)
    ap.add_argument("--dtype", default="bfloat16")
    ap.add_argument("--output", required=True)
    args = ap.parse_args(argv)
    if args.recipe:
        os.makedirs(args.output, exist_ok=True)
        model_type, config, parts, added = RECIPES[args.recipe](args)
        pad = max(args.pad_vocab_to, 64) if added else args.pad_vocab_to
        if args.skip_weights:
            with open(os.path.join(args.output, "config.json"), "w") as f:
                json.dump(config, f, indent=1)
            print(json.dumps({"config_only": True, "model_type": model_type, "added_tokens": added}))
            return {"config_only": True}
    else:
        if not (args.model_type and args.config):
            ap.error("give --recipe, or --model-type with --config")
        with open(args.config) as f:
            config = json.load(f)
        model_type, parts, added, pad = args.model_type, dict(p.split("=", 1) for p in args.part), args.add_tokens, args.pad_vocab_to
    model, report = assemble(model_type, config, parts, added, pad, getattr(torch, args.dtype))
    hf_io.save_pretrained(model, args.output)
    print(json.dumps(report))
    return report


if __name__ == "__main__":
    main()
