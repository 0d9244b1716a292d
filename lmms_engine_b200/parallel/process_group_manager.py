"""Rank layout, device meshes and process groups.

Semantics follow the reference manager (src/lmms_engine/parallel/process_group_manager.py:22-208):
the world is a ``(dp, pp, cp, tp)`` grid with TP fastest-varying; ``dp x cp`` flattens into
the ``fsdp`` axis; expert parallelism uses its own 2-D mesh
``(dp_shard_mod_ep, dp_shard_in_ep)`` flattened into ``fsdp`` and ``ep``; HSDP builds an
independent ``(hsdp_replicate, hsdp_shard)`` mesh; PP must be 1.

Unlike the reference, the coordinate arithmetic lives in a plain ``RankLayout`` that needs
no process group (so it is unit-testable and usable by launch-time validation), and the
communicators are the ones ``DeviceMesh`` already owns instead of a second set built by
enumeration.  The device type follows the backend (``cuda`` for NCCL, ``cpu`` for gloo).
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.distributed as dist
from torch.distributed.device_mesh import DeviceMesh, init_device_mesh


@dataclass(frozen=True)
class RankLayout:
    """Pure arithmetic over the (dp, pp, cp, tp) grid."""

    world_size: int
    tp: int = 1
    cp: int = 1
    pp: int = 1
    dp: int = 1
    ep: int = 1
    hsdp_shard: int = 0

    def __post_init__(self):
        if self.world_size != self.tp * self.cp * self.pp * self.dp:
            raise ValueError(
                f"World size ({self.world_size}) != TP ({self.tp}) * CP ({self.cp}) * PP ({self.pp}) * DP ({self.dp})"
            )
        if self.pp != 1:
            raise ValueError("PP size must be 1 for now")
        if self.ep > 1:
            if self.ep % (self.cp * self.tp) != 0 or (self.dp * self.cp * self.tp) % self.ep != 0:
                raise ValueError(f"ep_size {self.ep} does not tile dp*cp*tp = {self.dp * self.cp * self.tp}")
            if self.cp != 1:
                raise ValueError("Currently only support cp = 1 for EP")
        if self.hsdp_shard == 1:
            raise ValueError(
                "hsdp_shard_size=1 means pure DDP, which is not supported. Use 0 to disable HSDP, or >1 to enable it."
            )
        if self.hsdp_shard > 1:
            if self.ep != 1:
                raise ValueError("HSDP + EP is not supported")
            if (self.dp * self.cp) % self.hsdp_shard != 0:
                raise ValueError(f"dp*cp ({self.dp * self.cp}) must be divisible by hsdp_shard_size ({self.hsdp_shard})")

    @classmethod
    def from_degrees(cls, world_size: int, tp=None, cp=None, ep=None, hsdp_shard=None) -> "RankLayout":
        """Layout for the degrees of a training configuration (``None`` / 0 mean 1); the data-parallel
        degree is whatever of the world the model-parallel degrees leave."""
        tp, cp, ep = int(tp or 1), int(cp or 1), int(ep or 1)
        if tp < 1 or cp < 1 or ep < 1:
            raise ValueError(f"parallel degrees must be positive: tp_degree={tp}, sp_ulysses_degree={cp}, ep_degree={ep}")
        if world_size % (tp * cp):
            raise ValueError(f"{world_size} ranks cannot be split into groups of sp_ulysses_degree x tp_degree = {cp} x {tp}")
        return cls(world_size=world_size, tp=tp, cp=cp, pp=1, dp=world_size // (tp * cp), ep=ep, hsdp_shard=int(hsdp_shard or 0))

    def coords(self, rank: int):
        """(dp, pp, cp, tp) coordinates of ``rank``."""
        tp = rank % self.tp
        rest = rank // self.tp
        cp = rest % self.cp
        rest //= self.cp
        pp = rest % self.pp
        dp = rest // self.pp
        return dp, pp, cp, tp

    def rank_of(self, dp: int, pp: int, cp: int, tp: int) -> int:
        return ((dp * self.pp + pp) * self.cp + cp) * self.tp + tp

    def group_ranks(self, rank: int, axis: str) -> List[int]:
        dp, pp, cp, tp = self.coords(rank)
        if axis == "tp":
            return [self.rank_of(dp, pp, cp, t) for t in range(self.tp)]
        if axis == "cp":
            return [self.rank_of(dp, pp, c, tp) for c in range(self.cp)]
        if axis == "pp":
            return [self.rank_of(dp, p, cp, tp) for p in range(self.pp)]
        if axis == "dp":
            return [self.rank_of(d, pp, cp, tp) for d in range(self.dp)]
        if axis == "dp_cp":
            return [self.rank_of(d, pp, c, tp) for d in range(self.dp) for c in range(self.cp)]
        if axis == "ep":
            in_ep = self.ep // (self.cp * self.tp)
            base = (rank // in_ep) * in_ep
            return list(range(base, base + in_ep))
        raise KeyError(axis)

    @property
    def dp_shard_mod_ep(self) -> int:
        return self.dp * self.cp * self.tp // self.ep

    @property
    def dp_shard_in_ep(self) -> int:
        return self.ep // (self.cp * self.tp)


class ProcessGroupManager:
    def __init__(self, tp_size, cp_size, pp_size, dp_size, ep_size=1, hsdp_shard_size=0, device_type=None):
        self.global_rank = dist.get_rank()
        self.world_size = dist.get_world_size()
        self.local_rank = int(os.environ.get("LOCAL_RANK", self.global_rank % max(torch.cuda.device_count(), 1)))
        hsdp_shard_size = hsdp_shard_size or 0
        self.layout = RankLayout(self.world_size, tp_size, cp_size, pp_size, dp_size, ep_size, hsdp_shard_size)
        if device_type is None:
            device_type = "cuda" if dist.get_backend() == "nccl" else "cpu"
        self.device_type = device_type

        self.tp_size, self.cp_size, self.pp_size, self.dp_size, self.ep_size = tp_size, cp_size, pp_size, dp_size, ep_size
        self.hsdp_shard_size = hsdp_shard_size
        self.enable_hsdp = hsdp_shard_size > 1

        self.base_mesh = init_device_mesh(
            device_type, (dp_size, pp_size, cp_size, tp_size), mesh_dim_names=("dp", "pp", "cp", "tp")
        )
        self.device_mesh: DeviceMesh = self.base_mesh
        self.ep_mesh: Optional[DeviceMesh] = None
        if ep_size > 1:
            self.device_mesh = init_device_mesh(
                device_type,
                (self.layout.dp_shard_mod_ep, self.layout.dp_shard_in_ep),
                mesh_dim_names=("dp_shard_mod_ep", "dp_shard_in_ep"),
            )
            self.device_mesh["dp_shard_mod_ep", "dp_shard_in_ep"]._flatten(mesh_dim_name="fsdp")
            self.device_mesh["dp_shard_in_ep"]._flatten(mesh_dim_name="ep")
            self.ep_mesh = self.device_mesh["ep"]
        else:
            self.device_mesh["dp", "cp"]._flatten(mesh_dim_name="fsdp")
        self.ep_world_size = ep_size if ep_size > 1 else 1

        self.hsdp_mesh = None
        if self.enable_hsdp:
            self.hsdp_mesh = init_device_mesh(
                device_type,
                ((dp_size * cp_size) // hsdp_shard_size, hsdp_shard_size),
                mesh_dim_names=("hsdp_replicate", "hsdp_shard"),
            )

        self.dp_rank, self.pp_rank, self.cp_rank, self.tp_rank = self.layout.coords(self.global_rank)
        self.tp_group = self.base_mesh.get_group("tp")
        self.cp_group = self.base_mesh.get_group("cp")
        self.pp_group = self.base_mesh.get_group("pp")
        self.dp_group = self.base_mesh.get_group("dp")
        self.dp_cp_group = (
            self.base_mesh["dp", "cp"]._flatten(mesh_dim_name="dp_cp").get_group() if ep_size > 1
            else self.device_mesh["fsdp"].get_group()
        )
        self.ep_group = self.ep_mesh.get_group() if self.ep_mesh is not None else None
        self.world_group = dist.group.WORLD

        for axis in ("tp", "cp", "pp", "dp"):
            ids = self.layout.group_ranks(self.global_rank, axis)
            setattr(self, f"{axis}_group_ids", ids)
            setattr(self, f"{axis}_world_size", len(ids))
            setattr(self, f"{axis}_first_rank", ids[0])
            setattr(self, f"{axis}_last_rank", ids[-1])
        self.dp_cp_world_size = dp_size * cp_size

    def __str__(self):
        return f"TP({self.tp_size})-CP({self.cp_size})-PP({self.pp_size})-DP({self.dp_size})-EP({self.ep_size})-Rank({self.global_rank})"

    @property
    def enable_tp(self):
        return self.tp_size > 1

    @property
    def enable_cp(self):
        return self.cp_size > 1

    @property
    def enable_pp(self):
        return self.pp_size > 1

    @property
    def enable_ep(self):
        return self.ep_size > 1

    @property
    def enable_parallel(self):
        return self.enable_tp or self.enable_pp or self.enable_ep

    @property
    def fsdp_mesh(self) -> DeviceMesh:
        """Mesh to hand to ``fully_shard``: 2-D (replicate, shard) under HSDP, else 1-D."""
        if self.enable_hsdp:
            return self.hsdp_mesh
        return self.device_mesh["fsdp"]

    @property
    def tp_mesh(self) -> DeviceMesh:
        return self.base_mesh["tp"]


process_group_manager: Optional[ProcessGroupManager] = None


def setup_process_group_manager(tp_size, cp_size, pp_size, dp_size, ep_size=1, hsdp_shard_size=0, device_type=None):
    global process_group_manager
    process_group_manager = ProcessGroupManager(
        tp_size, cp_size, pp_size, dp_size, ep_size, hsdp_shard_size=hsdp_shard_size, device_type=device_type
    )
    return process_group_manager
