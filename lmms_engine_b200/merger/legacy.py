"""Legacy checkpoint merging (reference: tools/merge_fsdp.py:45-173).

``--type fsdp2``: per-rank ``.pt`` shards whose tensors are plain dim-0 slices (or DTensors) ->
one state dict.  ``--type hf``: a torch.distributed.checkpoint directory, read without a process
group.  ``--merge``: average the merged weights of every ``checkpoint-*`` under the input (model
soup).  Output is HF-style safetensors next to the input unless ``--output_dir`` is given.
"""
from __future__ import annotations

import argparse
import glob
import json
import os
import re
from pathlib import Path
from typing import Dict, List

import torch

from ..models import hf_io
from ..train import checkpoint as ckpt
from .consolidate import consolidate


def merge_fsdp2_dir(ckpt_dir: str) -> Dict[str, torch.Tensor]:
    sub = Path(ckpt_dir) / ckpt.MODEL_DIR
    base = sub if sub.is_dir() else Path(ckpt_dir)
    files = sorted(glob.glob(str(base / "model_world_size_*_rank_*.pt")), key=lambda f: int(re.search(r"rank_(\d+)", f).group(1)))
    if not files:
        raise FileNotFoundError(f"no model_world_size_*_rank_*.pt under {base}")
    shards = [torch.load(f, map_location="cpu", weights_only=False) for f in files]
    if any(hasattr(v, "placements") for v in shards[0].values()):
        return consolidate(shards)
    return {k: (torch.cat([s[k] for s in shards], 0) if shards[0][k].dim() > 0 else shards[0][k]) for k in shards[0]}


def merge_dcp_dir(ckpt_dir: str) -> Dict[str, torch.Tensor]:
    import torch.distributed.checkpoint as dcp
    from torch.distributed.checkpoint.metadata import TensorStorageMetadata

    reader = dcp.FileSystemReader(ckpt_dir)
    meta = reader.read_metadata()
    state = {k: torch.empty(m.size, dtype=m.properties.dtype) for k, m in meta.state_dict_metadata.items()
             if isinstance(m, TensorStorageMetadata)}
    dcp.load(state, storage_reader=reader, no_dist=True)
    return state


def soup(states: List[Dict[str, torch.Tensor]]) -> Dict[str, torch.Tensor]:
    out = {}
    for k, v in states[0].items():
        if v.is_floating_point():
            acc = v.double().clone()
            for s in states[1:]:
                acc += s[k].double()
            out[k] = (acc / len(states)).to(v.dtype)
        else:
            out[k] = v
    return out


def main(argv=None):
    ap = argparse.ArgumentParser(description="merge FSDP / DCP shards into HF safetensors")
    ap.add_argument("--input_dir", required=True, help="a checkpoint directory, or a run directory with checkpoint-* inside")
    ap.add_argument("--output_dir", default=None)
    ap.add_argument("--type", default="fsdp2", choices=["hf", "fsdp2"])
    ap.add_argument("--merge", action="store_true", help="average all checkpoints found (model soup)")
    ap.add_argument("--dtype", default="bfloat16")
    ap.add_argument("--step", type=int, default=None, help="merge checkpoint-<step> instead of the newest one")
    ap.add_argument("--state_dict_dirname", default=None, help="sub-directory holding the shards (default: pytorch_model_fsdp_0)")
    ap.add_argument("--model_name_or_class", default=None, help="accepted for compatibility; the config saved with the checkpoint is used")
    args = ap.parse_args(argv)
    one = merge_dcp_dir if args.type == "hf" else merge_fsdp2_dir
    inp = Path(args.input_dir)
    cands = ckpt.list_checkpoints(str(inp)) if any(inp.glob("checkpoint-*")) else [str(inp)]
    if args.step is not None:
        cands = [c for c in cands if c.rstrip("/").endswith(f"checkpoint-{args.step}")] or cands
    if args.state_dict_dirname:
        cands = [os.path.join(c, args.state_dict_dirname) if os.path.isdir(os.path.join(c, args.state_dict_dirname)) else c for c in cands]
    if not args.merge:
        cands = cands[-1:]
    states = [one(c) for c in cands]
    full = soup(states) if len(states) > 1 else states[0]
    dtype = getattr(torch, args.dtype)
    full = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in full.items()}
    out = Path(args.output_dir) if args.output_dir else Path(cands[-1]) / ("hf_soup" if len(states) > 1 else "hf")
    cfg_path = Path(cands[-1]) / "config.json"
    config = json.load(open(cfg_path)) if cfg_path.exists() else None
    hf_io.save_pretrained(full, str(out), config=config)
    print(out)
    return out


if __name__ == "__main__":
    main()
