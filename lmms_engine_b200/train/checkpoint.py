"""Checkpoint layout of the fsdp2 trainer, byte-compatible with the reference
(src/lmms_engine/train/fsdp2/fsdp2_trainer.py:499-612):

    checkpoint-{step}/pytorch_model_fsdp_0/model_world_size_{W}_rank_{r}.pt   DTensor state dict
    checkpoint-{step}/pytorch_ema_model_fsdp_0/...                            (EMA weights)
    checkpoint-{step}/optimizer/optimizer_world_size_{W}_rank_{r}.pt
    checkpoint-{step}/extra_state/extra_state_world_size_{W}_rank_{r}.pt
    checkpoint-{step}/dataloader_state/dataloader_state_world_size_{W}_rank_{r}.pt
    checkpoint-{step}/config.json (+ processor files, rank 0)

When parameters are replicated (owner-sharded runtime) each rank still writes only its
``Shard(0)`` slice wrapped as a DTensor, so the merger and the reference's tooling read
the files unchanged.  Unlike the reference, checkpoints can be loaded at a different world
size: the loader consolidates all rank files of the saved world size and re-slices.
"""
from __future__ import annotations

import glob
import os
import re
import shutil
from typing import Any, Dict, List, Optional

import torch
import torch.distributed as dist

from ..merger.consolidate import consolidate

MODEL_DIR = "pytorch_model_fsdp_0"
EMA_DIR = "pytorch_ema_model_fsdp_0"


def rank_file(kind: str, world: int, rank: int) -> str:
    return f"{kind}_world_size_{world}_rank_{rank}.pt"


def list_checkpoints(output_dir: str) -> List[str]:
    paths = [p for p in glob.glob(os.path.join(output_dir, "checkpoint-*")) if re.search(r"checkpoint-(\d+)$", p)]
    return sorted(paths, key=lambda p: int(p.rsplit("-", 1)[1]))


def latest_checkpoint(output_dir: str) -> Optional[str]:
    ck = list_checkpoints(output_dir)
    return ck[-1] if ck else None


def latest_resumable_checkpoint(output_dir: str) -> Optional[str]:
    """Newest checkpoint that finished saving.  Directories written by tools that leave no completion
    marker are accepted only if no checkpoint of the run has one."""
    from ..utils import failure

    ck = list_checkpoints(output_dir)
    if not ck:
        return None
    if not any(os.path.exists(os.path.join(p, failure.MARKER)) for p in ck):
        return ck[-1]
    return failure.latest_valid_checkpoint(output_dir, ck)


def rotate_checkpoints(output_dir: str, save_total_limit: Optional[int]) -> None:
    if not save_total_limit or save_total_limit <= 0:
        return
    ck = list_checkpoints(output_dir)
    for p in ck[: max(0, len(ck) - save_total_limit)]:
        shutil.rmtree(p, ignore_errors=True)


def shard0_dtensor_state(full_state: Dict[str, torch.Tensor], mesh) -> Dict[str, Any]:
    """Wrap this rank's dim-0 chunk of every (replicated) tensor as a ``Shard(0)`` DTensor."""
    from torch.distributed.tensor import DTensor, Shard

    world, rank = mesh.size(), mesh.get_local_rank()
    out: Dict[str, Any] = {}
    for k, v in full_state.items():
        v = v.detach()
        if v.dim() == 0:
            out[k] = v.cpu()
            continue
        chunks = list(torch.chunk(v, world, dim=0))
        if rank < len(chunks):
            local = chunks[rank].clone()  # own storage: DTensor pickling rejects offset views
        else:
            local = v.new_empty((0,) + tuple(v.shape[1:]))
        out[k] = DTensor.from_local(local.cpu() if mesh.device_type == "cpu" else local, mesh, [Shard(0)],
                                    run_check=False, shape=v.shape, stride=v.stride())
    return out


def save_rank_state(ckpt_dir: str, sub: str, kind: str, world: int, rank: int, obj: Any) -> str:
    d = os.path.join(ckpt_dir, sub)
    os.makedirs(d, exist_ok=True)
    path = os.path.join(d, rank_file(kind, world, rank))
    torch.save(obj, path)
    return path


def load_rank_state(ckpt_dir: str, sub: str, kind: str, world: int, rank: int) -> Any:
    path = os.path.join(ckpt_dir, sub, rank_file(kind, world, rank))
    return torch.load(path, map_location="cpu", weights_only=False)


def saved_world_size(ckpt_dir: str, sub: str = MODEL_DIR, kind: str = "model") -> int:
    files = glob.glob(os.path.join(ckpt_dir, sub, f"{kind}_world_size_*_rank_0.pt"))
    if not files:
        raise FileNotFoundError(f"no {kind} shards under {os.path.join(ckpt_dir, sub)}")
    return int(re.search(r"world_size_(\d+)_rank_0", files[0]).group(1))


def load_full_model_state(ckpt_dir: str, sub: str = MODEL_DIR) -> Dict[str, torch.Tensor]:
    """Consolidate every rank file of the saved world size into full tensors (CPU)."""
    world = saved_world_size(ckpt_dir, sub)
    shards = [load_rank_state(ckpt_dir, sub, "model", world, r) for r in range(world)]
    return consolidate(shards)


def barrier() -> None:
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.barrier()
