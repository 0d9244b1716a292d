"""Parameter-sharded data parallelism (ZeRO-3) for B200: ``sharding_runtime: native_sharded``.

The owner-sharded runtime keeps a full bf16 copy of the weights on every GPU, which stops at a
few tens of billions of parameters.  This runtime shards the weights as well.  What is stored and
where:

* every parameter of a repeated block (a decoder layer, a vision block: everything under a
  ``...<name>.<index>.`` module) has ONE owner rank; Muon matrices are dealt by Newton-Schulz cost,
  the block's other parameters by size.  The owner keeps the bf16 value, the fp32 master copy and
  the optimizer state in its ``own`` range; nobody else keeps anything.
* parameters outside such blocks (embeddings, output head, final norm) stay replicated and are
  updated on even slices, exactly as in the owner-sharded runtime ("resident" region).

One step, per block ``b`` (forward in order, backward in reverse):

    gather      the block's parameters are copied from their owners' ``own`` ranges into one of a few
                block-sized weight slots of this GPU (copy engines over NVLink on a prefetch stream,
                one copy per parameter, no multicast); block b+1 is fetched while block b computes;
                the GEMMs read the local slot, never a peer's memory
    release     after the block's forward (and again after its backward) the slot is free for reuse
    grad slot   before the block's backward its ``.grad`` tensors are pointed at a zeroed, peer-mapped
                gradient slot; when all of them are final, a side stream raises this rank's flag for
                the block, waits for the peers' flags, pulls the owned parameters' gradients from all
                peers' slots, adds the sum to the owner's fp32 gradient range and acknowledges the
                slot on every peer (a slot is rewritten only after all acknowledgements)
    update      as in the owner-sharded runtime, but nothing of a block is published: the next
                step's gather reads the owners' new values

The reference gets the same memory behaviour from FSDP2 ``fully_shard`` per decoder layer with
NCCL all-gather / reduce-scatter (src/lmms_engine/utils/fsdp2_utils.py:24-111,
src/lmms_engine/train/fsdp2/fsdp2_trainer.py:156-200) and gathers / scatters every Muon matrix once
more inside its optimizer (src/lmms_engine/utils/muon_utils.py:234-272); here whole-matrix
ownership is the sharding, so Newton-Schulz needs no extra exchange.

Two communication back ends: peer memory (``PeerShardComm``: NVLink, device flags, bounded waits)
and ``torch.distributed`` (``TorchShardComm``: broadcast from the owner / reduce to the owner; used
on CPU with gloo and as the fallback across hosts).
"""
from __future__ import annotations

import contextlib
import ctypes
import math
import os
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from ..ops import _cuda
from ..ops import muon as muon_ops
from ..ops import optim as optim_ops
from .owner_sharded import ALIGN, OwnerShardedRuntime, Segment, _round_up, lpt_assign


# ------------------------------------------------------------------------------------------------
# communication back ends
class TorchShardComm:
    """Gather = broadcast from the owner, reduce = ``dist.reduce`` to the owner.  Every rank issues the
    same collectives in the same order (the hooks that drive them fire in module order)."""

    peer = False

    def __init__(self, group):
        self.group = group
        self.n = dist.get_world_size(group) if group is not None else 1
        self.rank = dist.get_rank(group) if group is not None else 0

    def global_rank(self, r: int) -> int:
        return dist.get_global_rank(self.group, r) if self.group is not None else r

    def allocate(self, numel: int, dtype, device) -> torch.Tensor:
        return torch.zeros(max(numel, 1), dtype=dtype, device=device)

    def gather(self, dst: torch.Tensor, own: torch.Tensor, items: Sequence[Tuple[int, int, int, int]]) -> None:
        """items: (owner, offset in the owner's ``own`` buffer, offset in dst, numel)."""
        for owner, src_off, dst_off, numel in items:
            out = dst[dst_off : dst_off + numel]
            if owner == self.rank:
                out.copy_(own[src_off : src_off + numel])
            if self.n > 1:
                dist.broadcast(out, src=self.global_rank(owner), group=self.group)

    def reduce_slot(self, slot: torch.Tensor, slot_index: int, use: int, bucket: int, epoch: int,
                    items: Sequence[Tuple[int, int, int, int]], g_own: torch.Tensor) -> None:
        """items: (owner, offset in the slot, offset in the owner's gradient range, numel)."""
        for owner, slot_off, own_off, numel in items:
            part = slot[slot_off : slot_off + numel]
            if self.n > 1:
                dist.reduce(part, dst=self.global_rank(owner), group=self.group)
            if owner == self.rank:
                g_own[own_off : own_off + numel].add_(part.to(g_own.dtype))

    def wait_acks(self, slot_index: int, use: int) -> None:
        return  # the reduce above is complete when it returns

    def bump(self, key) -> int:
        c = self.__dict__.setdefault("_counters", {})
        c[key] = c.get(key, 0) + 1
        return c[key]

    def all_reduce_sum(self, t: torch.Tensor) -> None:
        if self.n > 1:
            dist.all_reduce(t, group=self.group)

    def barrier(self) -> None:
        if self.n > 1:
            dist.barrier(group=self.group)

    def broadcast_all(self, flat: torch.Tensor, src: int = 0) -> None:
        if self.n > 1:
            dist.broadcast(flat, src=self.global_rank(src), group=self.group)

    # resident region: same calls as owner_sharded.TorchComm
    def reduce_to_owner(self, grad_flat, ranges) -> None:
        if self.n == 1:
            return
        works = [dist.reduce(grad_flat[lo:hi], dst=self.global_rank(r), group=self.group, async_op=True)
                 for r in range(self.n) for lo, hi in ranges[r] if hi > lo]
        for w in works:
            w.wait()

    def publish(self, param_flat, ranges) -> None:
        if self.n == 1:
            return
        works = [dist.broadcast(param_flat[lo:hi], src=self.global_rank(r), group=self.group, async_op=True)
                 for r in range(self.n) for lo, hi in ranges[r] if hi > lo]
        for w in works:
            w.wait()


_cuda.register("b200_peer_memcpy", "peer_comm", "ppls")
_cuda.register("b200_peer_slot_reduce", "peer_comm", "ppipiiiipiipiiis")
_cuda.register("b200_peer_wait_flags", "peer_comm", "piiiipis")


class PeerShardComm:
    """Peer-memory back end on top of ``PeerComm`` (symmetric buffers, flag pad, bounded waits)."""

    peer = True
    ACK_OFFSET = 16  # inside a bucket's / slot's 32-word flag block: [0,16) ready, [16,32) acknowledgements

    def __init__(self, peer_comm):
        self.pc = peer_comm
        self.n, self.rank, self.group = peer_comm.n, peer_comm.rank, peer_comm.group
        self.device = peer_comm.device

    def allocate(self, numel: int, dtype, device) -> torch.Tensor:
        return self.pc.allocate(max(numel, 8), dtype, device)

    def _peer_ptrs(self, t: torch.Tensor):
        return self.pc._handles[t.data_ptr()][1].buffer_ptrs

    def gather(self, dst: torch.Tensor, own: torch.Tensor, items) -> None:
        ptrs = self._peer_ptrs(own)
        es = own.element_size()
        for owner, src_off, dst_off, numel in items:
            _cuda.call("b200_peer_memcpy", dst.data_ptr() + dst_off * es, int(ptrs[owner]) + src_off * es, numel * es,
                       _cuda.stream())

    def slot_flag_block(self, slot_index: int) -> int:
        # slots use the flag blocks after the buckets' (see ParamShardedRuntime._flag_block)
        return self.pc.BUCKET_FLAG_BASE + slot_index * self.pc.BUCKET_FLAG_STRIDE

    def reduce_slot(self, slot: torch.Tensor, slot_index: int, use: int, bucket: int, epoch: int, items, g_own) -> None:
        mine = [v for owner, slot_off, own_off, numel in items if owner == self.rank for v in (slot_off, own_off, numel)]
        arr = (ctypes.c_long * max(len(mine), 1))(*mine)
        pc = self.pc
        st = _cuda.status_word(self.device)
        _cuda.call("b200_peer_slot_reduce", ctypes.addressof(pc._peers(slot)), ctypes.addressof(pc._pad_ptrs), self.n, g_own.data_ptr(),
                   self.rank, int(slot.dtype == torch.float32), int(g_own.dtype == torch.float32),
                   pc.BUCKET_FLAG_BASE + bucket * pc.BUCKET_FLAG_STRIDE, ctypes.addressof(arr), len(mine) // 3, epoch & 0x7FFFFFFF,
                   st.data_ptr(), self.slot_flag_block(slot_index) + self.ACK_OFFSET, use & 0x7FFFFFFF, pc.BARRIER_TIMEOUT_MS,
                   _cuda.stream())

    def wait_acks(self, slot_index: int, use: int) -> None:
        pc = self.pc
        st = _cuda.status_word(self.device)
        _cuda.call("b200_peer_wait_flags", ctypes.addressof(pc._pad_ptrs), self.n, self.rank,
                   self.slot_flag_block(slot_index) + self.ACK_OFFSET, use & 0x7FFFFFFF, st.data_ptr(), pc.BARRIER_TIMEOUT_MS,
                   _cuda.stream())

    def bump(self, key) -> int:
        return self.pc.bump(key)

    def all_reduce_sum(self, t):
        self.pc.all_reduce_sum(t)

    def barrier(self):
        self.pc.barrier()

    def broadcast_all(self, flat, src: int = 0):
        self.pc.broadcast_all(flat, src)


# ------------------------------------------------------------------------------------------------
class ParamShardedRuntime(OwnerShardedRuntime):
    """ZeRO-3 flavour of the owner-sharded runtime (module docstring).  Same constructor; ``comm`` may be a
    ``PeerComm`` (wrapped into ``PeerShardComm``) or ``None`` (torch.distributed)."""

    WEIGHT_SLOTS = int(os.environ.get("LMMS_B200_WEIGHT_SLOTS", "3"))
    GRAD_SLOTS = int(os.environ.get("LMMS_B200_GRAD_SLOTS", "2"))

    def __init__(self, model, group=None, *, comm=None, **kw):
        self._sh_model = model
        self._res_comm = comm  # PeerComm (or None): drives the resident region like the owner-sharded runtime
        self.sc = PeerShardComm(comm) if comm is not None else TorchShardComm(group)
        super().__init__(model, group, comm=comm if comm is not None else None, **kw)

    # ---- layout ---------------------------------------------------------------------------------
    def _plan_and_allocate(self, params, use_muon: bool, muon_ns_steps: int, no_decay_patterns) -> None:
        n, rank = self.n, self.rank
        model = self._sh_model
        # which parameters live in a shardable block (a module reached by the bucket key)
        block_of: Dict[int, str] = {}
        for i, (nm, p) in enumerate(params):
            key = self.bucket_key(nm)
            is_block = key[-1:].isdigit() and "." in key
            if is_block:
                try:
                    model.get_submodule(key)
                except AttributeError:
                    is_block = False
            if is_block:
                block_of[i] = key
        stray = [nm for i, (nm, p) in enumerate(params) if i not in block_of and use_muon and muon_ops.is_muon_param(nm, p)]
        if stray and rank == 0:
            from ..utils.logging_utils import logger

            logger.warning(f"native_sharded: {len(stray)} Muon-eligible matrices lie outside a repeated block and are updated "
                           f"with AdamW in the replicated region: {stray[:4]}{' ...' if len(stray) > 4 else ''}")
        sh_idx = [i for i in range(len(params)) if i in block_of]
        mu_idx = [i for i in sh_idx if use_muon and muon_ops.is_muon_param(*params[i])]
        ad_idx = [i for i in sh_idx if i not in set(mu_idx)]
        owner_of: Dict[int, int] = {}
        owner_of.update(zip(mu_idx, lpt_assign([muon_ops.ns_flops(tuple(params[i][1].shape), muon_ns_steps) for i in mu_idx], n)))
        owner_of.update(zip(ad_idx, lpt_assign([float(params[i][1].numel()) for i in ad_idx], n)))

        def is_decay(nm, p):
            return p.ndim >= 2 and not any(pat in nm for pat in no_decay_patterns)

        # virtual flat layout: [rank0: matrices | adam decay | adam no-decay][rank1: ...]...[resident region]
        segs: List[Segment] = []
        self.own_span: List[Tuple[int, int]] = []       # whole owned range of every rank
        self.muon_ranges = []                           # its Muon part
        self.own_adam: List[Tuple[int, int, int]] = []  # (lo, end of the decayed part, hi) of its AdamW part
        off = 0
        for r in range(n):
            lo = off
            for i in mu_idx:
                if owner_of[i] == r:
                    nm, p = params[i]
                    segs.append(Segment(nm, tuple(p.shape), p.numel(), "muon", True, r, off))
                    off = _round_up(off + p.numel(), ALIGN)
            mu_end = off
            for want in (True, False):
                for i in ad_idx:
                    nm, p = params[i]
                    if owner_of[i] == r and is_decay(nm, p) == want:
                        segs.append(Segment(nm, tuple(p.shape), p.numel(), "adam", want, r, off))
                        off = _round_up(off + p.numel(), ALIGN)
                if want:
                    dec_end = off
            self.own_span.append((lo, off))
            self.muon_ranges.append((lo, mu_end))
            self.own_adam.append((mu_end, dec_end, off))
        res_lo = off
        for want in (True, False):
            for i, (nm, p) in enumerate(params):
                if i in block_of or is_decay(nm, p) != want:
                    continue
                segs.append(Segment(nm, tuple(p.shape), p.numel(), "adam", want, -1, off))
                off = _round_up(off + p.numel(), ALIGN)
            if want:
                self.adam_decay_end = off
        res_hi = off
        chunk = _round_up(max(1, math.ceil((res_hi - res_lo) / n)), ALIGN)
        self.res_lo = res_lo
        self.adam_ranges = [(res_lo + r * chunk, res_lo + (r + 1) * chunk) for r in range(n)]
        self.total = res_lo + chunk * n
        self.segments = segs
        self.by_name = {s.name: s for s in segs}
        self.block_key = {params[i][0]: k for i, k in block_of.items()}

        # ---- physical buffers -----------------------------------------------------------------------
        dev, pd = self.device, self.param_dtype
        own_max = max(hi - lo for lo, hi in self.own_span)
        self.P_own = self.sc.allocate(own_max, pd, dev)              # peer-mapped: the others gather from it
        self.G_own = torch.zeros(max(own_max, 1), dtype=torch.float32, device=dev)
        res_n = self.total - res_lo
        rc = self.comm                                              # resident region: owner-sharded machinery
        self.P = rc.allocate(res_n, pd, dev)                         # indexed by (virtual offset - res_lo)
        self.G = rc.allocate(res_n, self.grad_dtype, dev)
        self.bind_grads = self.grad_dtype == pd
        name_to_param = dict(params)
        self.params = name_to_param
        my_lo = self.own_span[rank][0]
        with torch.no_grad():
            for s in segs:
                p = name_to_param[s.name]
                if s.owner < 0:
                    view = self.P[s.offset - res_lo : s.offset - res_lo + s.numel].view(s.shape)
                    view.copy_(p.data)
                    p.data = view
                    p.grad = self.G[s.offset - res_lo : s.offset - res_lo + s.numel].view(s.shape) if self.bind_grads else None
        # sharded parameters: every rank starts from rank 0's values
        self._blocks: List[str] = []
        for s in segs:
            if s.owner >= 0 and self.block_key[s.name] not in self._blocks:
                self._blocks.append(self.block_key[s.name])
        self._block_segs: Dict[str, List[Segment]] = {k: [] for k in self._blocks}
        for s in segs:
            if s.owner >= 0:
                self._block_segs[self.block_key[s.name]].append(s)
        self._slot_off: Dict[str, int] = {}
        self.block_numel = 0
        for k, ss in self._block_segs.items():
            o = 0
            for s in ss:
                self._slot_off[s.name] = o
                o = _round_up(o + s.numel, ALIGN)
            self.block_numel = max(self.block_numel, o)
        with torch.no_grad():
            for s in segs:
                if s.owner < 0:
                    continue
                p = name_to_param[s.name]
                full = p.data.to(device=dev, dtype=pd).reshape(-1).contiguous()
                if n > 1:
                    dist.broadcast(full, src=dist.get_global_rank(self.sc.group, 0) if self.sc.group is not None else 0,
                                   group=self.sc.group)
                if s.owner == rank:
                    self.P_own[s.offset - my_lo : s.offset - my_lo + s.numel].copy_(full)
                p.data = torch.empty(0, dtype=pd, device=dev)
                p.grad = None
                del full
        self.comm.broadcast_all(self.P, 0)
        # ---- slots ------------------------------------------------------------------------------------
        self._w_slots = [torch.empty(max(self.block_numel, 1), dtype=pd, device=dev) for _ in range(self.WEIGHT_SLOTS)]
        self._g_slots = [self.sc.allocate(self.block_numel, pd, dev) for _ in range(self.GRAD_SLOTS)]
        cuda = dev.type == "cuda"
        self._prefetch = torch.cuda.Stream(device=dev) if (cuda and self.sc.peer) else None
        self._w_block: List[Optional[str]] = [None] * self.WEIGHT_SLOTS   # block whose weights the slot holds
        self._w_busy = [False] * self.WEIGHT_SLOTS                         # between ensure and release
        self._w_ready: List[Any] = [None] * self.WEIGHT_SLOTS
        self._w_free: List[Any] = [None] * self.WEIGHT_SLOTS
        self._w_clock = [0] * self.WEIGHT_SLOTS
        self._clock = 0
        self._g_next = 0
        self._g_use = [0] * self.GRAD_SLOTS
        self._g_of: Dict[str, Tuple[int, int]] = {}
        self._blk_round: Dict[str, int] = {k: 0 for k in self._blocks}
        self._blk_count: Dict[str, int] = {k: 0 for k in self._blocks}
        self._blk_index = {k: i for i, k in enumerate(self._blocks)}
        self._params_ready_ev = None
        self._install_block_hooks()

    # ---- flag blocks: buckets of the resident region first, then the blocks, then the gradient slots
    def _flag_block(self, block: str) -> int:
        return self.n_buckets + self._blk_index[block]

    def _slot_flag_index(self, j: int) -> int:
        return self.n_buckets + len(self._blocks) + j

    # ---- weights --------------------------------------------------------------------------------------
    def _in_backward(self) -> bool:
        try:
            return torch._C._current_graph_task_id() != -1
        except Exception:
            return False

    def _gather_into_slot(self, block: str) -> int:
        free = [j for j in range(self.WEIGHT_SLOTS) if not self._w_busy[j]]
        if not free:
            raise RuntimeError("no free weight slot: raise LMMS_B200_WEIGHT_SLOTS (blocks nested inside blocks?)")
        j = min(free, key=lambda q: (self._w_block[q] is not None, self._w_clock[q]))
        old = self._w_block[j]
        if old is not None:
            self._unbind(old)
        my_lo = {r: self.own_span[r][0] for r in range(self.n)}
        # parameters that this rank owns are used in place (ensure_block binds them to the own range)
        items = [(s.owner, s.offset - my_lo[s.owner], self._slot_off[s.name], s.numel) for s in self._block_segs[block]
                 if s.owner != self.rank or not self.sc.peer]
        if self._prefetch is not None:
            with torch.cuda.stream(self._prefetch):
                if self._w_free[j] is not None:
                    self._prefetch.wait_event(self._w_free[j])      # the slot's last reader has finished
                if self._params_ready_ev is not None:
                    self._prefetch.wait_event(self._params_ready_ev)  # the owners' values of this step are final
                self.sc.gather(self._w_slots[j], self.P_own, items)
                ev = torch.cuda.Event()
                ev.record(self._prefetch)
            self._w_ready[j] = ev
        else:
            self.sc.gather(self._w_slots[j], self.P_own, items)
            self._w_ready[j] = None
        self._w_block[j] = block
        return j

    def _slot_of(self, block: str) -> Optional[int]:
        for j in range(self.WEIGHT_SLOTS):
            if self._w_block[j] == block:
                return j
        return None

    def _unbind(self, block: str) -> None:
        for s in self._block_segs[block]:
            self.params[s.name].data = torch.empty(0, dtype=self.param_dtype, device=self.device)

    def ensure_block(self, block: str) -> None:
        """Make the block's parameters usable on the current stream (gathering them if no slot holds them)."""
        j = self._slot_of(block)
        if j is None:
            j = self._gather_into_slot(block)
        if self._w_ready[j] is not None:
            torch.cuda.current_stream(self.device).wait_event(self._w_ready[j])
        slot = self._w_slots[j]
        base = self.own_span[self.rank][0]
        for s in self._block_segs[block]:
            if s.owner == self.rank and self.sc.peer:
                self.params[s.name].data = self.P_own[s.offset - base : s.offset - base + s.numel].view(s.shape)
            else:
                o = self._slot_off[s.name]
                self.params[s.name].data = slot[o : o + s.numel].view(s.shape)
        self._w_busy[j] = True
        self._clock += 1
        self._w_clock[j] = self._clock

    def prefetch_block(self, block: Optional[str]) -> None:
        if block is None or self._slot_of(block) is not None or all(self._w_busy):
            return
        self._gather_into_slot(block)

    def release_block(self, block: str) -> None:
        j = self._slot_of(block)
        if j is None:
            return
        self._w_busy[j] = False
        if self.device.type == "cuda":
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream(self.device))
            self._w_free[j] = ev

    def _neighbour(self, block: str, step: int) -> Optional[str]:
        i = self._blk_index[block] + step
        return self._blocks[i] if 0 <= i < len(self._blocks) else None

    # ---- hooks ------------------------------------------------------------------------------------------
    def _install_block_hooks(self) -> None:
        model = self._sh_model
        for block in self._blocks:
            mod = model.get_submodule(block)
            mod.register_forward_pre_hook(self._make_pre_forward(block))
            mod.register_forward_hook(self._make_post_forward(block))
            mod.register_full_backward_pre_hook(self._make_pre_backward(block))
            for s in self._block_segs[block]:
                self.params[s.name].register_post_accumulate_grad_hook(self._make_grad_hook(block))

    def _make_pre_forward(self, block):
        def hook(mod, args):
            self.ensure_block(block)
            if not self._in_backward():
                self.prefetch_block(self._neighbour(block, +1))
        return hook

    def _make_post_forward(self, block):
        def hook(mod, args, out):
            if not self._in_backward():  # a recomputation inside backward keeps the weights for the backward itself
                self.release_block(block)
        return hook

    def _make_pre_backward(self, block):
        def hook(mod, grad_output):
            self.ensure_block(block)
            self.prefetch_block(self._neighbour(block, -1))
            self._bind_grad_slot(block)
        return hook

    def _bind_grad_slot(self, block: str) -> None:
        if block in self._g_of:
            return
        j = self._g_next
        self._g_next = (j + 1) % self.GRAD_SLOTS
        if self._g_use[j] > 0:
            self.sc.wait_acks(self._slot_flag_index(j), self._g_use[j])  # every owner has read the slot's last content
        self._g_use[j] = self.sc.bump(("slot", self._slot_flag_index(j)))
        slot = self._g_slots[j]
        slot.zero_()
        for s in self._block_segs[block]:
            o = self._slot_off[s.name]
            self.params[s.name].grad = slot[o : o + s.numel].view(s.shape)
        self._g_of[block] = (j, self._g_use[j])
        self._blk_count[block] = 0

    def _make_grad_hook(self, block):
        n_params = len(self._block_segs[block])

        def hook(p):
            if block not in self._g_of:
                return
            self._blk_count[block] += 1
            if self._blk_count[block] == n_params:
                self._reduce_block(block)
        return hook

    def _reduce_block(self, block: str) -> None:
        """All gradients of the block are final on this rank: hand them to their owners."""
        j, use = self._g_of.pop(block)
        self._blk_round[block] = self.sc.bump(("block", self._flag_block(block)))
        my_lo = {r: self.own_span[r][0] for r in range(self.n)}
        items = [(s.owner, self._slot_off[s.name], s.offset - my_lo[s.owner], _round_up(s.numel, 8)) for s in self._block_segs[block]]
        if self._side is not None:
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream(self.device))
            self._side.wait_event(ev)
            with torch.cuda.stream(self._side):
                self.sc.reduce_slot(self._g_slots[j], self._slot_flag_index(j), use, self._flag_block(block), self._blk_round[block],
                                    items, self.G_own)
        else:
            self.sc.reduce_slot(self._g_slots[j], self._slot_flag_index(j), use, self._flag_block(block), self._blk_round[block],
                                items, self.G_own)
        for s in self._block_segs[block]:
            self.params[s.name].grad = None
        self.release_block(block)

    def after_backward(self) -> None:
        """Call after every backward pass: blocks of which only some parameters received a gradient."""
        for block in list(self._g_of):
            self._reduce_block(block)

    # ---- buckets of the resident region ------------------------------------------------------------------
    def _build_buckets(self) -> None:
        sharded = [s for s in self.segments if s.owner >= 0]
        self.segments = [s for s in self.segments if s.owner < 0]      # what the base class buckets and binds
        shift = self.res_lo
        for s in self.segments:
            s.offset -= shift
        self.adam_ranges = [(lo - shift, hi - shift) for lo, hi in self.adam_ranges]
        self.adam_decay_end -= shift
        super()._build_buckets()
        self.sharded_segments = sharded
        if self._side is None and self.device.type == "cuda" and self.sc.peer:
            self._side = torch.cuda.Stream(device=self.device)

    # ---- step ---------------------------------------------------------------------------------------------
    @torch.no_grad()
    def step(self, lr_factor: float = 1.0) -> torch.Tensor:
        sc = self.sc
        self.after_backward()
        if self.overlap:
            self._finish_reduce()
        elif self._side is not None:
            done = torch.cuda.Event()
            done.record(self._side)
            torch.cuda.current_stream(self.device).wait_event(done)
        self.step_count += 1
        if not self.overlap:
            self.comm.reduce_to_owner(self.G, self.all_ranges)
        inv_n = 1.0 / self.n
        span = self.own_span[self.rank]
        n_own = span[1] - span[0]
        first = True
        if n_own > 0:
            optim_ops.sumsq_(self.G_own[:n_own], self._sumsq, accumulate=False)
            first = False
        lo, hi = self.adam_ranges[self.rank]
        if hi > lo:
            optim_ops.sumsq_(self.G[lo:hi], self._sumsq, accumulate=not first)
            first = False
        if first:
            self._sumsq.zero_()
        sc.all_reduce_sum(self._sumsq)
        if inv_n != 1.0:
            self._sumsq.mul_(inv_n * inv_n)
        optim_ops.clip_coef(self._sumsq, self._norm, self._coef, self._skip, float(self.max_grad_norm or 0.0))
        gscale = self._coef * inv_n if inv_n != 1.0 else self._coef
        lr = self.lr * lr_factor
        self._adam_update(lr, gscale)          # resident slice (published to the replicas)
        self._own_adam_update(lr, gscale)      # this rank's block parameters that are not Muon matrices
        self._muon_update(lr, gscale)
        if self.overlap:
            self.comm.barrier()
        else:
            self.comm.publish(self.P, self.all_ranges)
            sc.barrier()
        self.G.zero_()
        self.G_own.zero_()
        # the weight slots hold last step's values
        for j in range(self.WEIGHT_SLOTS):
            if self._w_block[j] is not None:
                self._unbind(self._w_block[j])
            self._w_block[j] = None
            self._w_busy[j] = False
        if self.device.type == "cuda":
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream(self.device))
            self._params_ready_ev = ev
        return self._norm

    @property
    def all_ranges(self):
        return [[self.adam_ranges[r]] for r in range(self.n)]

    def _own_adam_update(self, lr, gscale) -> None:
        lo, split, hi = self.own_adam[self.rank]
        base = self.own_span[self.rank][0]
        for a, b, wd in ((lo, split, self.weight_decay), (split, hi, 0.0)):
            if b <= a:
                continue
            s = slice(a - lo, b - lo)
            optim_ops.adamw_step(
                self.oa_master[s], self.P_own[a - base : b - base] if self.needs_master else None, self.oa_m[s], self.oa_v[s],
                self.G_own[a - base : b - base], lr=lr, beta1=self.betas[0], beta2=self.betas[1], eps=self.eps, wd=wd,
                step=self.step_count, gscale=gscale, skip=self._skip,
            )

    def _muon_update(self, lr, gscale) -> None:
        lo = self.muon_ranges[self.rank][0]
        base = self.own_span[self.rank][0]
        cfg = self.muon

        def body(s: Segment, lane) -> None:
            a, b = s.offset, s.offset + s.numel
            x = torch.empty(s.shape, dtype=torch.bfloat16 if self.P_own.is_cuda else torch.float32, device=self.device)
            optim_ops.muon_momentum(self.mu_mom[a - lo : b - lo], self.G_own[a - base : b - base], x.view(-1), lane["sumsq"],
                                    beta=cfg["momentum"], nesterov=cfg["nesterov"], gscale=gscale)
            o = muon_ops.orthogonalize(x, cfg["ns_steps"], lane["work"], max_ctas=lane["ctas"])
            if lane["stream"] is not None:
                x.record_stream(lane["stream"])
            optim_ops.muon_update(
                self.mu_master[a - lo : b - lo], self.P_own[a - base : b - base] if self.needs_master else None, o.reshape(-1),
                lr=lr, wd=self.weight_decay, scale=muon_ops.muon_scale(s.shape, cfg["rms_scale"]), skip=self._skip,
            )

        self._on_lanes(self.my_matrices, body)

    # ---- owned state --------------------------------------------------------------------------------------
    def _init_owned_state(self) -> None:
        f32 = dict(dtype=torch.float32, device=self.device)
        rank = self.rank
        base = self.own_span[rank][0]
        mu_lo, mu_hi = self.muon_ranges[rank]
        a_lo, _, a_hi = self.own_adam[rank]
        self.needs_master = self.param_dtype != torch.float32
        own = self.P_own
        self.mu_master = own[mu_lo - base : mu_hi - base].float() if self.needs_master else own[mu_lo - base : mu_hi - base]
        self.mu_mom = torch.zeros(mu_hi - mu_lo, **f32)
        self.oa_master = own[a_lo - base : a_hi - base].float() if self.needs_master else own[a_lo - base : a_hi - base]
        self.oa_m = torch.zeros(a_hi - a_lo, **f32)
        self.oa_v = torch.zeros(a_hi - a_lo, **f32)
        r_lo, r_hi = self.adam_ranges[rank]
        self.ad_master = self.P[r_lo:r_hi].float() if self.needs_master else self.P[r_lo:r_hi]
        self.ad_m = torch.zeros(r_hi - r_lo, **f32)
        self.ad_v = torch.zeros(r_hi - r_lo, **f32)
        self.own_ranges = []
        self.my_matrices = [s for s in self.sharded_segments if s.kind == "muon" and s.owner == rank]

    # ---- whole-model views (checkpoints, evaluation) ---------------------------------------------------------
    @torch.no_grad()
    def full_state_items(self):
        """Yield ``(name, full tensor)`` for every parameter, gathering the sharded ones block by block
        (the tensor of a sharded parameter is only valid until the next item is requested)."""
        for s in self.segments:
            yield s.name, self.params[s.name].data
        for block in self._blocks:
            self.ensure_block(block)
            if self.device.type == "cuda":
                torch.cuda.current_stream(self.device).synchronize()
            for s in self._block_segs[block]:
                yield s.name, self.params[s.name].data
            self.release_block(block)

    @torch.no_grad()
    def load_full_state(self, full: Dict[str, torch.Tensor]) -> None:
        """Overwrite parameters from a full state dict (every rank holds the same ``full``)."""
        base = self.own_span[self.rank][0]
        for s in self.segments:
            if s.name in full:
                self.params[s.name].data.copy_(full[s.name].to(self.param_dtype))
        for s in self.sharded_segments:
            if s.name in full and s.owner == self.rank:
                self.P_own[s.offset - base : s.offset - base + s.numel].copy_(full[s.name].reshape(-1).to(self.param_dtype))
        for j in range(self.WEIGHT_SLOTS):
            if self._w_block[j] is not None:
                self._unbind(self._w_block[j])
            self._w_block[j] = None
            self._w_busy[j] = False
        self.sc.barrier()

    def refresh_master_from_params(self) -> None:
        if not self.needs_master:
            return
        rank = self.rank
        base = self.own_span[rank][0]
        mu_lo, mu_hi = self.muon_ranges[rank]
        a_lo, _, a_hi = self.own_adam[rank]
        self.mu_master.copy_(self.P_own[mu_lo - base : mu_hi - base])
        self.oa_master.copy_(self.P_own[a_lo - base : a_hi - base])
        r_lo, r_hi = self.adam_ranges[rank]
        self.ad_master.copy_(self.P[r_lo:r_hi])

    def state_dict(self) -> Dict[str, Any]:
        sd = super().state_dict()
        sd.update({"sharded": True, "own_span": self.own_span[self.rank], "oa_master": self.oa_master.detach().cpu() if self.needs_master else None,
                   "oa_m": self.oa_m.cpu(), "oa_v": self.oa_v.cpu(),
                   "segments": [(s.name, s.shape, s.kind, s.owner, s.offset) for s in self.segments + self.sharded_segments]})
        return sd

    def load_state_dict(self, sd: Dict[str, Any]) -> None:
        super().load_state_dict(sd)
        self.oa_m.copy_(sd["oa_m"])
        self.oa_v.copy_(sd["oa_v"])
        if self.needs_master:
            self.oa_master.copy_(sd["oa_master"])

    def zero_grad(self) -> None:
        self.G.zero_()
        self.G_own.zero_()
