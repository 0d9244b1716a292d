"""``Muon`` as a ``torch.optim.Optimizer`` for the stock-FSDP2 path (DTensor parameters on a
1-D mesh) and for single-device use.  Parameter groups carry ``use_muon``; Muon groups take
``lr, momentum, weight_decay, nesterov, ns_steps, rms_scale``, the others are Adam groups with
``lr, betas, eps, weight_decay`` (same group contract as the reference optimizer,
src/lmms_engine/utils/muon_utils.py:331-482).

For sharded parameters the momentum lives on the local shard; the Newton-Schulz input is
all-gathered, the matrix is orthogonalised on ONE owner rank (round-robin by parameter
index, like the reference's ``index % world``) and broadcast back, and every rank applies its
slice.  The engine's own runtime (``parallel/owner_sharded.py``) avoids these per-parameter
collectives altogether by making whole matrices the unit of sharding.
"""
from __future__ import annotations

from typing import Any, Dict

import torch
import torch.distributed as dist

from ..ops import muon as muon_ops


def _is_dtensor(t) -> bool:
    return hasattr(t, "_local_tensor") and hasattr(t, "placements")


class Muon(torch.optim.Optimizer):
    def __init__(self, param_groups, defaults=None):
        defaults = dict(defaults or {"lr": 0.02})
        groups = []
        for g in param_groups:
            g = dict(g)
            if "use_muon" not in g:
                raise ValueError("every param group needs 'use_muon'")
            if g["use_muon"]:
                g.setdefault("lr", 0.02)
                g.setdefault("momentum", 0.95)
                g.setdefault("weight_decay", 0.0)
                g.setdefault("rms_scale", True)
                g.setdefault("nesterov", True)
                g.setdefault("ns_steps", 5)
            else:
                g.setdefault("lr", 3e-4)
                g.setdefault("betas", (0.9, 0.95))
                g.setdefault("eps", 1e-10)
                g.setdefault("weight_decay", 0.0)
            groups.append(g)
        super().__init__(groups, defaults)

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        index = 0
        for group in self.param_groups:
            for p in group["params"]:
                if p.grad is None:
                    continue
                if group["use_muon"]:
                    self._muon_param(p, group, index)
                    index += 1
                else:
                    self._adam_param(p, group)
        return loss

    # ------------------------------------------------------------------ Adam branch
    def _adam_param(self, p, group):
        st = self.state[p]
        g = p.grad._local_tensor if _is_dtensor(p.grad) else p.grad
        w = p._local_tensor if _is_dtensor(p) else p
        if not st:
            st["step"] = 0
            st["m"] = torch.zeros_like(w, dtype=torch.float32)
            st["v"] = torch.zeros_like(w, dtype=torch.float32)
        st["step"] += 1
        b1, b2 = group["betas"]
        gf = g.float()
        st["m"].lerp_(gf, 1 - b1)
        st["v"].lerp_(gf * gf, 1 - b2)
        mh = st["m"] / (1 - b1 ** st["step"])
        vh = st["v"] / (1 - b2 ** st["step"])
        w.mul_(1 - group["lr"] * group["weight_decay"])
        w.add_((mh / (vh.sqrt() + group["eps"])).to(w.dtype), alpha=-group["lr"])

    # ------------------------------------------------------------------ Muon branch
    def _muon_param(self, p, group, index):
        st = self.state[p]
        sharded = _is_dtensor(p)
        g = p.grad._local_tensor if sharded else p.grad
        w = p._local_tensor if sharded else p
        if "momentum" not in st:
            st["momentum"] = torch.zeros_like(w, dtype=torch.float32)
        mom = st["momentum"]
        gf = g.float()
        mom.lerp_(gf, 1 - group["momentum"])
        upd = gf.lerp(mom, group["momentum"]) if group["nesterov"] else mom
        full_shape = tuple(p.shape)
        if sharded:
            from torch.distributed.tensor import DTensor

            mesh = p.device_mesh
            pg = mesh.get_group()
            world, me = dist.get_world_size(pg), dist.get_rank(pg)
            full = DTensor.from_local(upd.to(torch.bfloat16 if upd.is_cuda else torch.float32), mesh, p.placements,
                                      run_check=False, shape=p.shape, stride=p.stride()).full_tensor()
            owner = index % world
            if me == owner:
                out = self._orthogonalize(full.reshape(full_shape[0], -1), group).reshape(full_shape).to(full.dtype).contiguous()
            else:
                out = torch.empty_like(full)
            dist.broadcast(out, src=dist.get_global_rank(pg, owner), group=pg)
            # this rank's slice of the update, in the layout of its shard
            shard_dim = next((pl.dim for pl in p.placements if pl.is_shard()), None)
            if shard_dim is None:
                local = out
            else:
                chunk = -(-full_shape[shard_dim] // world)
                start = min(me * chunk, full_shape[shard_dim])
                local = out.narrow(shard_dim, start, w.shape[shard_dim])
        else:
            local = self._orthogonalize(upd.reshape(full_shape[0], -1), group).reshape(full_shape)
        scale = muon_ops.muon_scale((full_shape[0], max(1, int(torch.tensor(full_shape[1:]).prod()))), group["rms_scale"])
        w.mul_(1 - group["lr"] * group["weight_decay"])
        w.add_(local.to(w.dtype), alpha=-group["lr"] * scale)

    @staticmethod
    def _orthogonalize(u: torch.Tensor, group: Dict[str, Any]) -> torch.Tensor:
        x = u.to(torch.bfloat16) if u.is_cuda else u.float()
        x = x / (x.float().norm() + 1e-7).to(x.dtype)
        return muon_ops.newton_schulz(x.contiguous(), group["ns_steps"])
