"""Assemble the initial checkpoint of a composite model from the checkpoints of its parts.

    python -m lmms_engine_b200.tools.prepare_init_weight --model-type aero --config aero_config.json \\
        --part language_model=Qwen2.5-7B-Instruct --part audio_tower=Qwen2-Audio-7B/audio_tower \\
        --add-tokens 3 --pad-vocab-to 64 --output ./aero_init

Every ``--part PREFIX=DIR`` loads a safetensors / ``pytorch_model.bin`` directory and places its tensors under
``PREFIX`` of the new model (the part's own ``model.`` / hub prefixes are tried as they are and with the common
wrappers stripped); parameters that no part covers keep the model's initialisation (projectors, merger).  When the
vocabulary grows, the new embedding and output rows are drawn from a Gaussian fitted to the existing rows with the
covariance scaled by 1e-5, so new tokens start near the mean embedding.

One generic tool for what the reference spreads over its per-family scripts
(tools/prepare_init_weight/prepare_aero.py:44-133, prepare_rae_siglip2.py, prepare_aero_omni.py).
"""
from __future__ import annotations

import argparse
import json
from typing import Dict, List, Tuple

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


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--model-type", required=True)
    ap.add_argument("--config", required=True, help="json file with the composite model's configuration")
    ap.add_argument("--part", action="append", default=[], help="PREFIX=DIR, repeatable")
    ap.add_argument("--add-tokens", type=int, default=0)
    ap.add_argument("--pad-vocab-to", type=int, default=1)
    ap.add_argument("--dtype", default="bfloat16")
    ap.add_argument("--output", required=True)
    args = ap.parse_args(argv)
    with open(args.config) as f:
        config = json.load(f)
    parts = dict(p.split("=", 1) for p in args.part)
    model, report = assemble(args.model_type, config, parts, args.add_tokens, args.pad_vocab_to, getattr(torch, args.dtype))
    hf_io.save_pretrained(model, args.output)
    print(json.dumps(report))
    return report


if __name__ == "__main__":
    main()
