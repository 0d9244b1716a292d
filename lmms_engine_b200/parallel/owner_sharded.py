"""Owner-sharded data parallelism: the engine's native ZeRO runtime for B200.

A B200 has 180 GB of HBM, so for models up to a few tens of billions of parameters the
bf16 working copy of the weights fits on every GPU.  This runtime therefore keeps the bf16
parameters REPLICATED (no all-gather before forward, no re-gather in backward, nothing
on the critical path of the step) and shards what is actually large: fp32 master weights,
optimizer moments and the optimizer's compute.  One step is

    forward/backward      gradients accumulate in a flat buffer (bf16, or fp32 on request)
    reduce-to-owner       every rank receives the summed gradient of the ranges it owns; with the
                          peer-memory implementation this happens bucket by bucket (one bucket per
                          decoder layer) on a side stream WHILE the backward of the earlier layers
                          is still running, so only the last bucket's transfer is exposed
    norm / clip           sum of squares over owned ranges, one scalar all-reduce
    owner update          AdamW on an even slice of the elementwise region; Muon on WHOLE
                          matrices, spread over ranks by Newton-Schulz cost (LPT)
    publish               owners write the new bf16 values into every replica; with the
                          peer-memory implementation the update kernels store them into all
                          replicas themselves, matrix by matrix, next to the Newton-Schulz chains
                          of the other matrices

Whole-matrix ownership is what Muon needs (Newton-Schulz works on full matrices): the
reference gathers FSDP shards to ``index % world`` owners and scatters them back with
NCCL gather/scatter per parameter (src/lmms_engine/utils/muon_utils.py:206-275); here the
ownership is the sharding itself.  The collective steps go through a ``Comm`` object: the
default uses torch.distributed (NCCL or gloo); on NVLink systems the peer-memory
implementation in ``parallel/peer_comm.py`` reads and writes peer memory directly from its own
kernels (bucketed pull-reduce, update + publish in one kernel).  The Muon momentum is NOT folded
into the reduce: it needs the clip coefficient, which exists only once every bucket is reduced.

For models too large to replicate, the trainer falls back to stock FSDP2
(``sharding_runtime: torch_fsdp2``), as the reference does everywhere
(src/lmms_engine/utils/fsdp2_utils.py:24-111).
"""
from __future__ import annotations

import contextlib
import math
import os
import re
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from ..ops import muon as muon_ops
from ..ops import optim as optim_ops

ALIGN = 64  # elements; keeps every parameter 128-byte aligned for TMA and vector access


def _round_up(x: int, a: int) -> int:
    return (x + a - 1) // a * a


@dataclass
class Segment:
    name: str
    shape: Tuple[int, ...]
    numel: int
    kind: str  # "muon" | "adam"
    decay: bool
    owner: int  # muon: owning rank; adam: -1 (evenly sliced)
    offset: int = 0  # into the flat buffers


def lpt_assign(costs: Sequence[float], n: int) -> List[int]:
    """Longest-processing-time assignment: heaviest item first onto the least loaded rank."""
    order = sorted(range(len(costs)), key=lambda i: (-costs[i], i))
    load = [0.0] * n
    owner = [0] * len(costs)
    for i in order:
        r = min(range(n), key=lambda k: (load[k], k))
        owner[i] = r
        load[r] += costs[i]
    return owner


class TorchComm:
    """Collective steps of the runtime on torch.distributed (NCCL / gloo)."""

    supports_overlap = False

    def __init__(self, group):
        self.group = group
        self.n = dist.get_world_size(group) if group is not None else 1
        self.rank = dist.get_rank(group) if group is not None else 0

    def global_rank(self, r: int) -> int:
        return dist.get_global_rank(self.group, r) if self.group is not None else r

    def allocate(self, numel: int, dtype, device) -> torch.Tensor:
        return torch.zeros(numel, dtype=dtype, device=device)

    def reduce_to_owner(self, grad_flat: torch.Tensor, ranges: List[List[Tuple[int, int]]]) -> None:
        """Sum ``grad_flat[lo:hi]`` of all ranks into rank r for every (lo, hi) in ranges[r]."""
        if self.n == 1:
            return
        works = []
        for r in range(self.n):
            for lo, hi in ranges[r]:
                if hi > lo:
                    works.append(dist.reduce(grad_flat[lo:hi], dst=self.global_rank(r), group=self.group, async_op=True))
        for w in works:
            w.wait()

    def publish(self, param_flat: torch.Tensor, ranges: List[List[Tuple[int, int]]]) -> None:
        if self.n == 1:
            return
        works = []
        for r in range(self.n):
            for lo, hi in ranges[r]:
                if hi > lo:
                    works.append(dist.broadcast(param_flat[lo:hi], src=self.global_rank(r), group=self.group, async_op=True))
        for w in works:
            w.wait()

    def broadcast_all(self, flat: torch.Tensor, src: int = 0) -> None:
        if self.n > 1:
            dist.broadcast(flat, src=self.global_rank(src), group=self.group)

    def all_reduce_sum(self, t: torch.Tensor) -> None:
        if self.n > 1:
            dist.all_reduce(t, group=self.group)

    def barrier(self) -> None:
        if self.n > 1:
            dist.barrier(group=self.group)


class OwnerShardedRuntime:
    """Flat replicated parameters + owner-sharded optimizer (AdamW and Muon)."""

    def __init__(
        self,
        model: torch.nn.Module,
        group=None,
        *,
        lr: float,
        weight_decay: float = 0.0,
        betas: Tuple[float, float] = (0.9, 0.999),
        eps: float = 1e-8,
        max_grad_norm: float = 1.0,
        use_muon: bool = False,
        muon_momentum: float = 0.95,
        muon_nesterov: bool = True,
        muon_ns_steps: int = 5,
        muon_rms_scale: bool = True,
        param_dtype: torch.dtype = torch.bfloat16,
        grad_dtype: Optional[torch.dtype] = None,
        device: Optional[torch.device] = None,
        comm: Optional[Any] = None,
        no_decay_patterns: Sequence[str] = ("bias", "norm"),
    ):
        self.model = model
        self.comm = comm if comm is not None else TorchComm(group)
        self.n, self.rank = self.comm.n, self.comm.rank
        self.lr, self.weight_decay, self.betas, self.eps = lr, weight_decay, betas, eps
        self.max_grad_norm = max_grad_norm
        self.muon = dict(momentum=muon_momentum, nesterov=muon_nesterov, ns_steps=muon_ns_steps, rms_scale=muon_rms_scale)
        self.param_dtype = param_dtype
        self.grad_dtype = grad_dtype or param_dtype
        self.step_count = 0
        self.breakdown = os.environ.get("LMMS_B200_STEP_BREAKDOWN", "0") == "1"
        self.phase_events: List[Tuple[str, Any]] = []
        self._ns_work: Dict[Any, torch.Tensor] = {}
        self._lanes = None

        params: List[Tuple[str, torch.nn.Parameter]] = []
        seen = set()
        for name, p in model.named_parameters():
            if id(p) in seen or not p.requires_grad:
                continue
            seen.add(id(p))
            params.append((name, p))
        self.device = device or params[0][1].device

        self._plan_and_allocate(params, use_muon, muon_ns_steps, no_decay_patterns)
        self._build_buckets()
        self._init_owned_state()
        f32 = dict(dtype=torch.float32, device=self.device)
        self._sumsq = torch.zeros(1, **f32)
        self._norm = torch.zeros(1, **f32)
        self._coef = torch.ones(1, **f32)
        self._skip = torch.zeros(1, dtype=torch.int32, device=self.device)

    def _plan_and_allocate(self, params, use_muon: bool, muon_ns_steps: int, no_decay_patterns) -> None:
        """Ownership, the flat layout and the flat buffers; binds every parameter to its slice."""
        param_dtype = self.param_dtype
        muon_idx = [i for i, (nm, p) in enumerate(params) if use_muon and muon_ops.is_muon_param(nm, p)]
        owners = lpt_assign([muon_ops.ns_flops(tuple(params[i][1].shape), muon_ns_steps) for i in muon_idx], self.n)
        owner_of = dict(zip(muon_idx, owners))

        # ---- flat layout: [rank0 matrices | rank1 matrices | ... | adam decay | adam no-decay]
        segs: List[Segment] = []
        self.muon_ranges: List[Tuple[int, int]] = []
        off = 0
        for r in range(self.n):
            lo = off
            for i in muon_idx:
                if owner_of[i] != r:
                    continue
                nm, p = params[i]
                segs.append(Segment(nm, tuple(p.shape), p.numel(), "muon", True, r, off))
                off = _round_up(off + p.numel(), ALIGN)
            self.muon_ranges.append((lo, off))
        adam_lo = off
        for want_decay in (True, False):
            for i, (nm, p) in enumerate(params):
                if i in owner_of:
                    continue
                decay = p.ndim >= 2 and not any(pat in nm for pat in no_decay_patterns)
                if decay != want_decay:
                    continue
                segs.append(Segment(nm, tuple(p.shape), p.numel(), "adam", decay, -1, off))
                off = _round_up(off + p.numel(), ALIGN)
            if want_decay:
                self.adam_decay_end = off
        adam_hi = off
        chunk = _round_up(max(1, math.ceil((adam_hi - adam_lo) / self.n)), ALIGN)
        total = adam_lo + chunk * self.n
        self.adam_ranges = [(adam_lo + r * chunk, adam_lo + (r + 1) * chunk) for r in range(self.n)]
        self.total = total
        self.segments = segs
        self.by_name = {s.name: s for s in segs}

        # ---- flat buffers and parameter views -------------------------------------------------
        self.P = self.comm.allocate(total, param_dtype, self.device)
        self.G = self.comm.allocate(total, self.grad_dtype, self.device)
        # gradients accumulate straight into the flat buffer when it has the parameters' dtype; an fp32
        # buffer under bf16 parameters is fed by a hook that adds each finished gradient and drops it
        self.bind_grads = self.grad_dtype == param_dtype
        name_to_param = dict(params)
        with torch.no_grad():
            for s in segs:
                p = name_to_param[s.name]
                view = self.P[s.offset : s.offset + s.numel].view(s.shape)
                view.copy_(p.data)
                p.data = view
                p.grad = self.G[s.offset : s.offset + s.numel].view(s.shape) if self.bind_grads else None
        self.params = name_to_param
        # replicas must start identical whatever each rank's initialisation did
        self.comm.broadcast_all(self.P, 0)

    def _init_owned_state(self) -> None:
        """fp32 master weights and optimizer moments of the ranges this rank owns."""
        my_mu, my_ad = self.muon_ranges[self.rank], self.adam_ranges[self.rank]
        self.own_ranges = [my_mu, my_ad]
        f32 = dict(dtype=torch.float32, device=self.device)
        self.needs_master = self.param_dtype != torch.float32
        self.mu_master = self.P[my_mu[0] : my_mu[1]].float() if self.needs_master else self.P[my_mu[0] : my_mu[1]]
        self.mu_mom = torch.zeros(my_mu[1] - my_mu[0], **f32)
        self.ad_master = self.P[my_ad[0] : my_ad[1]].float() if self.needs_master else self.P[my_ad[0] : my_ad[1]]
        self.ad_m = torch.zeros(my_ad[1] - my_ad[0], **f32)
        self.ad_v = torch.zeros(my_ad[1] - my_ad[0], **f32)
        self.my_matrices = [s for s in self.segments if s.kind == "muon" and s.owner == self.rank]

    # ---- gradient buckets ---------------------------------------------------------------------
    @staticmethod
    def bucket_key(name: str) -> str:
        """Parameters of one repeated block (``...layers.12.``) share a bucket; everything else is
        grouped by its first two name components (embeddings, final norm, output head)."""
        m = re.match(r"^(.*?\.\d+)\.", name)
        if m:
            return m.group(1)
        return ".".join(name.split(".")[:2])

    def _build_buckets(self) -> None:
        """Buckets in parameter order; ``bucket_ranges[b][r]`` = ranges of bucket b that rank r owns."""
        self.overlap = bool(getattr(self.comm, "supports_overlap", False)) and self.n > 1 and self.P.is_cuda \
            and os.environ.get("LMMS_B200_OVERLAP_REDUCE", "1") != "0"
        keys: Dict[str, int] = {}
        self.bucket_of: Dict[str, int] = {}
        for s in self.segments:
            self.bucket_of[s.name] = keys.setdefault(self.bucket_key(s.name), len(keys))
        nb = len(keys)
        if self.overlap and nb > self.comm.max_buckets:
            # fold the surplus into the last bucket rather than refuse the model
            for k in self.bucket_of:
                self.bucket_of[k] = min(self.bucket_of[k], self.comm.max_buckets - 1)
            nb = self.comm.max_buckets
        self.n_buckets = nb
        self.bucket_size = [0] * nb
        raw: List[List[List[Tuple[int, int]]]] = [[[] for _ in range(self.n)] for _ in range(nb)]
        for s in self.segments:
            b = self.bucket_of[s.name]
            self.bucket_size[b] += 1
            lo, hi = s.offset, _round_up(s.offset + s.numel, ALIGN)
            if s.kind == "muon":
                raw[b][s.owner].append((lo, hi))
            else:
                for r, (a0, a1) in enumerate(self.adam_ranges):
                    x0, x1 = max(lo, a0), min(hi, a1)
                    if x1 > x0:
                        raw[b][r].append((x0, x1))
        self.bucket_ranges = [[self._merge(rs) for rs in per_rank] for per_rank in raw]
        self._armed = False
        self._count = [0] * nb
        self._fired = [False] * nb
        self._side = torch.cuda.Stream(device=self.device) if self.overlap else None
        if self.overlap or not self.bind_grads:
            for s in self.segments:
                self.params[s.name].register_post_accumulate_grad_hook(self._make_hook(s))

    @staticmethod
    def _merge(ranges: List[Tuple[int, int]]) -> List[Tuple[int, int]]:
        out: List[Tuple[int, int]] = []
        for lo, hi in sorted(ranges):
            if out and lo <= out[-1][1]:
                out[-1] = (out[-1][0], max(out[-1][1], hi))
            else:
                out.append((lo, hi))
        return out

    def _make_hook(self, seg: "Segment"):
        b = self.bucket_of[seg.name]

        def hook(p):
            if not self.bind_grads and p.grad is not None:
                self.G[seg.offset : seg.offset + seg.numel].add_(p.grad.reshape(-1))
                p.grad = None
            if self.overlap and self._armed:
                self._count[b] += 1
                if self._count[b] == self.bucket_size[b] and not self._fired[b]:
                    self._fire(b, max_blocks=self.REDUCE_BLOCKS)

        return hook

    REDUCE_BLOCKS = int(os.environ.get("LMMS_B200_REDUCE_BLOCKS", "24"))

    def arm(self) -> None:
        """Call before the LAST backward of an optimizer step: from then on every bucket is reduced to
        its owners as soon as its gradients are final, next to the rest of the backward pass."""
        if self.overlap:
            self._armed = True
            self._count = [0] * self.n_buckets
            self._fired = [False] * self.n_buckets
            self._epoch = None

    def _fire(self, b: int, max_blocks: int) -> None:
        main = torch.cuda.current_stream(self.device)
        ev = torch.cuda.Event()
        ev.record(main)
        self._side.wait_event(ev)
        if getattr(self, "_epoch", None) is None:
            self._epoch = self.comm.bump("bucket_epoch")  # one epoch per optimizer step, the same on every rank
        with torch.cuda.stream(self._side):
            self.comm.bucket_reduce(self.G, b, self.bucket_ranges[b][self.rank], self._epoch, max_blocks)
        self._fired[b] = True

    def _finish_reduce(self) -> None:
        """Reduce whatever the backward hooks have not (parameters without a gradient this step, or a
        step that was not armed) and make the main stream wait for all of it."""
        for b in range(self.n_buckets):
            if not self._fired[b]:
                self._fire(b, max_blocks=0)
        done = torch.cuda.Event()
        done.record(self._side)
        torch.cuda.current_stream(self.device).wait_event(done)
        self._armed = False
        self._fired = [False] * self.n_buckets
        self._epoch = None

    # ------------------------------------------------------------------------------------
    @property
    def all_ranges(self) -> List[List[Tuple[int, int]]]:
        return [[self.muon_ranges[r], self.adam_ranges[r]] for r in range(self.n)]

    def zero_grad(self) -> None:
        self.G.zero_()

    def after_backward(self) -> None:
        """Called by the trainer after every backward pass (nothing to do when parameters are replicated)."""

    def rebind_grads(self) -> None:
        """Point every ``p.grad`` at its slice of the flat buffer again (after an external ``zero_grad(set_to_none)``)."""
        if not self.bind_grads:
            return
        for s in self.segments:
            self.params[s.name].grad = self.G[s.offset : s.offset + s.numel].view(s.shape)

    @torch.no_grad()
    def _mark(self, name: str) -> None:
        """Phase marker on the current stream (``LMMS_B200_STEP_BREAKDOWN=1``): the device time between two markers is the
        phase's exposed time.  Collected per step in ``phase_events``; ``phase_times()`` turns them into milliseconds."""
        if self.breakdown and self.P.is_cuda:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self.phase_events.append((name, ev))

    def phase_times(self) -> Dict[str, float]:
        """Milliseconds of every phase of the last step (synchronises)."""
        if not self.phase_events:
            return {}
        torch.cuda.synchronize()
        out: Dict[str, float] = {}
        for (_, a), (name, b) in zip(self.phase_events[:-1], self.phase_events[1:]):
            out[name] = out.get(name, 0.0) + a.elapsed_time(b)
        return out

    def step(self, lr_factor: float = 1.0) -> torch.Tensor:
        """Reduce, clip, update and publish.  Returns the global gradient norm (device scalar)."""
        comm = self.comm
        self._mark("backward")  # everything since the step's first marker (set by the trainer) up to here
        if self.overlap:
            self._finish_reduce()  # buckets were (mostly) reduced during the backward pass
            self.step_count += 1
        else:
            self.step_count += 1
            comm.reduce_to_owner(self.G, self.all_ranges)
        self._mark("reduce_exposed")
        # gradient of the MEAN loss over ranks; folded into the clip coefficient below
        inv_n = 1.0 / self.n
        first = True
        for lo, hi in self.own_ranges:
            if hi > lo:
                optim_ops.sumsq_(self.G[lo:hi], self._sumsq, accumulate=not first)
                first = False
        if first:
            self._sumsq.zero_()
        comm.all_reduce_sum(self._sumsq)
        if inv_n != 1.0:
            self._sumsq.mul_(inv_n * inv_n)
        optim_ops.clip_coef(self._sumsq, self._norm, self._coef, self._skip, float(self.max_grad_norm or 0.0))
        self._mark("grad_norm")
        gscale = self._coef * inv_n if inv_n != 1.0 else self._coef
        lr = self.lr * lr_factor
        self._adam_update(lr, gscale)
        self._mark("adamw_publish" if self.overlap else "adamw")
        self._muon_update(lr, gscale)
        self._mark("muon_publish" if self.overlap else "muon")
        if self.overlap:
            comm.barrier()  # every replica is complete, and every peer has finished reading my gradients
        else:
            comm.publish(self.P, self.all_ranges)
        self._mark("final_barrier" if self.overlap else "publish")
        self.G.zero_()
        self._mark("zero_grads")
        return self._norm

    def _adam_update(self, lr: float, gscale: torch.Tensor) -> None:
        lo, hi = self.adam_ranges[self.rank]
        if hi <= lo:
            return
        split = min(max(self.adam_decay_end, lo), hi)
        for a, b, wd in ((lo, split, self.weight_decay), (split, hi, 0.0)):
            if b <= a:
                continue
            s = slice(a - lo, b - lo)
            if self.overlap and self.needs_master:
                self.comm.adamw_publish(self.P, a, self.ad_master[s], self.ad_m[s], self.ad_v[s], self.G[a:b], lr=lr,
                                        beta1=self.betas[0], beta2=self.betas[1], eps=self.eps, wd=wd, step=self.step_count,
                                        gscale=gscale, skip=self._skip)
                continue
            optim_ops.adamw_step(
                self.ad_master[s], self.P[a:b] if self.needs_master else None, self.ad_m[s], self.ad_v[s], self.G[a:b],
                lr=lr, beta1=self.betas[0], beta2=self.betas[1], eps=self.eps, wd=wd, step=self.step_count,
                gscale=gscale, skip=self._skip,
            )
            if self.overlap:
                self.comm.publish_range(self.P, a, b)

    def _muon_update(self, lr: float, gscale: torch.Tensor) -> None:
        """Momentum, Newton-Schulz and the update of every matrix this rank owns.

        On CUDA the matrices are dealt round-robin to ``muon_lanes`` streams and every GEMM of a lane
        is confined to ``SMs / lanes`` CTAs: the symmetric products of one matrix have too few tiles
        for the whole GPU (210 upper-triangle tiles for a 3584 x 3584 product, 5 for a 512-row KV
        projection), so running several chains side by side on part of the SMs each removes most of
        the idle tail of every launch.  The chains are independent; the lanes join before the
        parameters are published."""
        lo, _ = self.muon_ranges[self.rank]
        cfg = self.muon

        def body(s: Segment, lane) -> None:
            a, b = s.offset, s.offset + s.numel
            mom = self.mu_mom[a - lo : b - lo]
            x = torch.empty(s.shape, dtype=torch.bfloat16 if self.P.is_cuda else torch.float32, device=self.device)
            optim_ops.muon_momentum(mom, self.G[a:b], x.view(-1), lane["sumsq"], beta=cfg["momentum"],
                                    nesterov=cfg["nesterov"], gscale=gscale)
            o = muon_ops.orthogonalize(x, cfg["ns_steps"], lane["work"], max_ctas=lane["ctas"])
            if lane["stream"] is not None:
                x.record_stream(lane["stream"])
            if self.overlap and self.needs_master and s.numel % 8 == 0:
                # update + publish in one kernel, on this lane, next to the other lanes' chains
                self.comm.muon_update_publish(self.P, a, self.mu_master[a - lo : b - lo], o.reshape(-1), lr=lr,
                                              wd=self.weight_decay, scale=muon_ops.muon_scale(s.shape, cfg["rms_scale"]),
                                              skip=self._skip, max_blocks=self.PUBLISH_BLOCKS)
                return
            optim_ops.muon_update(
                self.mu_master[a - lo : b - lo], self.P[a:b] if self.needs_master else None, o.reshape(-1),
                lr=lr, wd=self.weight_decay, scale=muon_ops.muon_scale(s.shape, cfg["rms_scale"]), skip=self._skip,
            )
            if self.overlap:
                self.comm.publish_range(self.P, a, _round_up(b, ALIGN))

        self._on_lanes(self.my_matrices, body)

    def _on_lanes(self, matrices, body) -> None:
        """Run ``body(segment, lane)`` for every matrix, dealt round-robin to the lanes' streams; the
        lanes start after what is queued on the current stream and the current stream waits for them."""
        lanes = self._muon_lanes()
        n_l = len(lanes)
        main = torch.cuda.current_stream() if n_l > 1 else None
        if n_l > 1:
            ready = torch.cuda.Event()
            ready.record(main)
            for lane in lanes:
                lane["stream"].wait_event(ready)
        for i, s in enumerate(matrices):
            lane = lanes[i % n_l]
            ctx = torch.cuda.stream(lane["stream"]) if n_l > 1 else contextlib.nullcontext()
            with ctx:
                body(s, lane)
        if n_l > 1:
            for lane in lanes:
                done = torch.cuda.Event()
                done.record(lane["stream"])
                main.wait_event(done)

    PUBLISH_BLOCKS = int(os.environ.get("LMMS_B200_PUBLISH_BLOCKS", "32"))

    def _muon_lanes(self):
        if self._lanes is None:
            n = 1
            if self.P.is_cuda:
                n = max(1, int(os.environ.get("LMMS_B200_MUON_LANES", "4")))
            sms = torch.cuda.get_device_properties(self.device).multi_processor_count if self.P.is_cuda else 0
            self._lanes = []
            for i in range(n):
                self._lanes.append({
                    "stream": torch.cuda.Stream(device=self.device) if n > 1 else None,
                    "sumsq": torch.zeros(1, dtype=torch.float32, device=self.device) if n > 1 else self._sumsq,
                    "work": {} if n > 1 else self._ns_work,
                    "ctas": (sms + n - 1) // n if n > 1 else 0,
                })
        return self._lanes

    # ---- checkpoint ------------------------------------------------------------------------
    def state_dict(self) -> Dict[str, Any]:
        return {
            "step": self.step_count,
            "world_size": self.n,
            "rank": self.rank,
            "muon_range": self.muon_ranges[self.rank],
            "adam_range": self.adam_ranges[self.rank],
            "mu_master": self.mu_master.detach().cpu() if self.needs_master else None,
            "mu_mom": self.mu_mom.cpu(),
            "ad_master": self.ad_master.detach().cpu() if self.needs_master else None,
            "ad_m": self.ad_m.cpu(),
            "ad_v": self.ad_v.cpu(),
            "segments": [(s.name, s.shape, s.kind, s.owner, s.offset) for s in self.segments],
        }

    def load_state_dict(self, sd: Dict[str, Any]) -> None:
        if sd["world_size"] != self.n or sd["rank"] != self.rank:
            raise ValueError("optimizer shard belongs to a different world size / rank")
        self.step_count = int(sd["step"])
        self.mu_mom.copy_(sd["mu_mom"])
        self.ad_m.copy_(sd["ad_m"])
        self.ad_v.copy_(sd["ad_v"])
        if self.needs_master:
            self.mu_master.copy_(sd["mu_master"])
            self.ad_master.copy_(sd["ad_master"])

    def refresh_master_from_params(self) -> None:
        """Re-derive fp32 masters from the (just loaded) parameter values."""
        if not self.needs_master:
            return
        my_mu, my_ad = self.own_ranges
        self.mu_master.copy_(self.P[my_mu[0] : my_mu[1]])
        self.ad_master.copy_(self.P[my_ad[0] : my_ad[1]])
