"""Merge a sharded training checkpoint into HF safetensors.

``FSDP2Merger`` reads ``pytorch_model_fsdp_0`` (or ``pytorch_ema_model_fsdp_0`` for
``checkpoint_type="ema"``) under a ``checkpoint-N`` directory (the newest one when given an
output directory), consolidates the per-rank DTensor shards, casts to bf16, re-ties tied
weights, and writes ``config.json`` + safetensors (+ processor files) that load in
``transformers``.  Reference: src/lmms_engine/merger/fsdp2.py:28-403.
"""
from __future__ import annotations

import glob
import json
import os
import re
import shutil
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path
from typing import Dict, List, Optional

import torch

from ..models import hf_io
from ..train import checkpoint as ckpt
from ..utils.logging_utils import logger
from .base import CheckpointMerger
from .consolidate import consolidate


class FSDP2Merger(CheckpointMerger):
    def __init__(self, checkpoint_path: str, output_path: Optional[str] = None, checkpoint_type: str = "regular",
                 model_general_type: Optional[str] = None, dtype: torch.dtype = torch.bfloat16, num_workers: int = 8):
        super().__init__(checkpoint_path, output_path)
        if checkpoint_type not in ("regular", "ema"):
            raise ValueError("checkpoint_type must be 'regular' or 'ema'")
        self.checkpoint_type = checkpoint_type
        self.model_general_type = model_general_type
        self.dtype = dtype
        self.num_workers = num_workers

    # -- locating ------------------------------------------------------------------------
    def resolve_checkpoint_path(self) -> Path:
        p = self.checkpoint_path
        if re.search(r"checkpoint-\d+$", str(p)):
            return p
        latest = ckpt.latest_checkpoint(str(p))
        if latest is None:
            if (p / ckpt.MODEL_DIR).is_dir():
                return p
            raise FileNotFoundError(f"no checkpoint-* directory under {p}")
        return Path(latest)

    @property
    def shard_dir_name(self) -> str:
        return ckpt.EMA_DIR if self.checkpoint_type == "ema" else ckpt.MODEL_DIR

    # -- loading -------------------------------------------------------------------------
    def load_shards(self, ckpt_dir: Path) -> List[Dict[str, torch.Tensor]]:
        sub = self.shard_dir_name
        world = ckpt.saved_world_size(str(ckpt_dir), sub)

        def _load(r):
            return ckpt.load_rank_state(str(ckpt_dir), sub, "model", world, r)

        with ThreadPoolExecutor(max_workers=min(self.num_workers, world)) as ex:
            return list(ex.map(_load, range(world)))

    # -- merge ---------------------------------------------------------------------------
    def merge(self) -> Path:
        ckpt_dir = self.resolve_checkpoint_path()
        shards = self.load_shards(ckpt_dir)
        if self.checkpoint_type == "ema":
            # EMA shards hold local tensors of the averaged parameters; lay them over the
            # placements recorded in the regular shards
            reg = ckpt.load_rank_state  # noqa: F841
            world = len(shards)
            regular = [ckpt.load_rank_state(str(ckpt_dir), ckpt.MODEL_DIR, "model", world, r) for r in range(world)]
            for r in range(world):
                for k, v in shards[r].items():
                    tpl = regular[r].get(k)
                    if hasattr(tpl, "placements") and not hasattr(v, "placements"):
                        from torch.distributed.tensor import DTensor

                        shards[r][k] = DTensor.from_local(v, tpl.device_mesh, tpl.placements, run_check=False,
                                                          shape=tpl.shape, stride=tpl.stride())
                for k, tpl in regular[r].items():
                    shards[r].setdefault(k, tpl)  # parameters outside the EMA filter
        full = consolidate(shards)
        full = {k: (v.to(self.dtype) if v.is_floating_point() else v) for k, v in full.items()}
        cfg_path = ckpt_dir / "config.json"
        config = json.load(open(cfg_path)) if cfg_path.exists() else None
        out = self.output_path or (ckpt_dir / ("hf_ema" if self.checkpoint_type == "ema" else "hf"))
        full = self.export_names(full, config)
        hf_io.save_pretrained(full, str(out), config=config)
        for fn in glob.glob(str(ckpt_dir / "*")):
            base = os.path.basename(fn)
            if os.path.isfile(fn) and base != "config.json" and not base.endswith((".pt", ".safetensors")):
                shutil.copy(fn, out / base)  # tokenizer / processor files
        logger.info(f"merged {len(shards)} shard(s) from {ckpt_dir} into {out}")
        return Path(out)

    def export_names(self, state: Dict[str, torch.Tensor], config: Optional[dict]) -> Dict[str, torch.Tensor]:
        """Native -> hub parameter naming (e.g. fused MoE experts back to per-expert tensors)."""
        model_type = (config or {}).get("model_type")
        try:
            from ..mapping_func import MODEL_REGISTRY
            from .. import models  # noqa: F401

            for _, (_, model_cls) in (MODEL_REGISTRY.get(model_type) or {}).items():
                if hasattr(model_cls, "export_hf_state_dict_static"):
                    return model_cls.export_hf_state_dict_static(state, config)
        except Exception as e:  # pragma: no cover
            logger.warning(f"name export skipped: {e}")
        return state
