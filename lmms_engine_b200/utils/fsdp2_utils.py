"""Helpers around stock FSDP2: wrapping, full-state load, gradient clipping across meshes
(reference: src/lmms_engine/utils/fsdp2_utils.py:24-111, 235-315).

``fsdp2_clip_grad_norm_`` differs from the reference on purpose: when parameters live on
several meshes (FSDP x EP, FSDP x TP) the reference clips each mesh group by ITS OWN norm
(:274-289); here one global norm is formed first and every group is scaled by the same
coefficient, which is what gradient clipping means.
"""
from __future__ import annotations

from typing import Dict, Iterable, List

import torch
import torch.distributed as dist


def _mesh_key(p) -> int:
    g = p.grad
    return id(g.device_mesh) if hasattr(g, "device_mesh") else 0


@torch.no_grad()
def fsdp2_clip_grad_norm_(parameters: Iterable[torch.nn.Parameter], max_norm: float, norm_type: float = 2.0) -> torch.Tensor:
    params = [p for p in parameters if p.grad is not None]
    if not params:
        return torch.zeros(())
    groups: Dict[int, List[torch.nn.Parameter]] = {}
    for p in params:
        groups.setdefault(_mesh_key(p), []).append(p)
    total_sq = None
    for ps in groups.values():
        grads = [p.grad for p in ps]
        n = torch.nn.utils.get_total_norm(grads, norm_type=norm_type, error_if_nonfinite=False)
        if hasattr(n, "full_tensor"):
            n = n.full_tensor()
        sq = n.float() ** 2
        total_sq = sq if total_sq is None else total_sq + sq.to(total_sq.device)
    total = total_sq.sqrt()
    if max_norm is not None and max_norm > 0:
        for ps in groups.values():
            torch.nn.utils.clip_grads_with_norm_(ps, max_norm, total)
    return total


def apply_fsdp2(model: torch.nn.Module, wrap_class_names, mesh, mp_policy=None, reshard_after_forward: bool = True):
    """``fully_shard`` every module whose class name is listed, untied embeddings, then the root."""
    from torch.distributed.fsdp import fully_shard

    kw = dict(mesh=mesh, reshard_after_forward=reshard_after_forward)
    if mp_policy is not None:
        kw["mp_policy"] = mp_policy
    names = set(wrap_class_names or [])
    tied = bool(getattr(getattr(model, "config", None), "tie_word_embeddings", False))
    for m in model.modules():
        if type(m).__name__ in names or (isinstance(m, torch.nn.Embedding) and not tied):
            fully_shard(m, **kw)
    fully_shard(model, **kw)
    return model


def fsdp2_load_full_state_dict(model: torch.nn.Module, full_state: Dict[str, torch.Tensor], device) -> None:
    """Load a full (unsharded) state dict into an FSDP2 model; rank 0 holds the values and
    the others receive them by broadcast."""
    from torch.distributed.checkpoint.state_dict import StateDictOptions, set_model_state_dict

    opts = StateDictOptions(full_state_dict=True, broadcast_from_rank0=dist.is_initialized() and dist.get_world_size() > 1)
    if dist.is_initialized() and dist.get_rank() != 0:
        full_state = {}
    set_model_state_dict(model, full_state, options=opts)
    for name, buf in model.named_buffers():
        if dist.is_initialized() and dist.get_world_size() > 1:
            dist.broadcast(buf.data, src=0)
