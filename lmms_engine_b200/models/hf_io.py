"""HF-compatible checkpoint IO for the native models: ``config.json`` plus (sharded)
safetensors with the upstream parameter names, so that what this engine writes loads in
``transformers`` and vice versa.  The reference gets this from ``PreTrainedModel``
(src/lmms_engine/train/runner.py:65-107, src/lmms_engine/merger/fsdp2.py:385-401)."""
from __future__ import annotations

import json
import os
from typing import Dict, Iterable, Optional

import torch

WEIGHTS_NAME = "model.safetensors"
INDEX_NAME = "model.safetensors.index.json"


def _safetensors():
    import safetensors.torch as st

    return st


def read_state_dict(path: str) -> Dict[str, torch.Tensor]:
    st = _safetensors()
    index = os.path.join(path, INDEX_NAME)
    out: Dict[str, torch.Tensor] = {}
    if os.path.exists(index):
        with open(index) as f:
            files = sorted(set(json.load(f)["weight_map"].values()))
        for fn in files:
            out.update(st.load_file(os.path.join(path, fn)))
        return out
    single = os.path.join(path, WEIGHTS_NAME)
    if os.path.exists(single):
        return st.load_file(single)
    legacy = os.path.join(path, "pytorch_model.bin")
    if os.path.exists(legacy):
        return torch.load(legacy, map_location="cpu", weights_only=True)
    raise FileNotFoundError(f"no weights found under {path}")


def load_pretrained_weights(model: torch.nn.Module, path: str, strict: bool = True) -> None:
    sd = read_state_dict(path)
    if hasattr(model, "convert_hf_state_dict"):
        sd = model.convert_hf_state_dict(sd)
    own = model.state_dict()
    tied = getattr(getattr(model, "config", None), "tie_word_embeddings", False)
    if tied and "lm_head.weight" not in sd and "model.embed_tokens.weight" in sd:
        sd["lm_head.weight"] = sd["model.embed_tokens.weight"]
    missing = [k for k in own if k not in sd]
    unexpected = [k for k in sd if k not in own]
    if strict and (missing or unexpected):
        raise KeyError(f"state dict mismatch: missing={missing[:8]} unexpected={unexpected[:8]}")
    model.load_state_dict({k: v for k, v in sd.items() if k in own}, strict=False)


def save_pretrained(
    model_or_state: "torch.nn.Module | Dict[str, torch.Tensor]",
    path: str,
    config: Optional[dict] = None,
    max_shard_bytes: int = 5 * 1024**3,
    tied: Iterable[str] = ("lm_head.weight",),
) -> None:
    """Write ``config.json`` and safetensors shards (tensors are made contiguous, tied
    duplicates are dropped as HF does)."""
    st = _safetensors()
    os.makedirs(path, exist_ok=True)
    if isinstance(model_or_state, torch.nn.Module):
        model = model_or_state
        state = model.state_dict()
        if hasattr(model, "export_hf_state_dict"):
            state = model.export_hf_state_dict(state)
        cfg = getattr(model, "config", None)
        if config is None and cfg is not None:
            config = cfg.to_dict() if hasattr(cfg, "to_dict") else dict(cfg)
        is_tied = bool(getattr(cfg, "tie_word_embeddings", False))
    else:
        state = dict(model_or_state)
        is_tied = bool((config or {}).get("tie_word_embeddings", False))
    if is_tied:
        for k in tied:
            state.pop(k, None)
    state = {k: v.detach().to("cpu").contiguous() for k, v in state.items()}
    shards, cur, cur_bytes = [], {}, 0
    for k, v in state.items():
        nb = v.numel() * v.element_size()
        if cur and cur_bytes + nb > max_shard_bytes:
            shards.append(cur)
            cur, cur_bytes = {}, 0
        cur[k] = v
        cur_bytes += nb
    if cur:
        shards.append(cur)
    if len(shards) == 1:
        st.save_file(shards[0], os.path.join(path, WEIGHTS_NAME), metadata={"format": "pt"})
    else:
        weight_map, total = {}, 0
        for i, sh in enumerate(shards):
            fn = f"model-{i + 1:05d}-of-{len(shards):05d}.safetensors"
            st.save_file(sh, os.path.join(path, fn), metadata={"format": "pt"})
            for k, v in sh.items():
                weight_map[k] = fn
                total += v.numel() * v.element_size()
        with open(os.path.join(path, INDEX_NAME), "w") as f:
            json.dump({"metadata": {"total_size": total}, "weight_map": weight_map}, f, indent=2)
    if config is not None:
        with open(os.path.join(path, "config.json"), "w") as f:
            json.dump(config, f, indent=2, default=str)
