"""Peer-memory implementation of the owner-sharded runtime's collective steps.

The flat parameter and gradient buffers are allocated from torch's symmetric-memory pool and
mapped into every rank of the group (NVLink / NVSwitch).

* ``bucket_reduce``: the gradients of one bucket (a decoder layer) are reduced to their owners
  while the backward pass of the remaining layers is still running: one kernel on a side stream
  raises this rank's per-bucket flag on every peer, waits (bounded) for the peers' flags and PULLS
  the owned ranges from all peers, summing in fp32.
* ``adamw_publish`` / ``muon_update_publish``: the owner's optimizer update writes the new bf16
  value of every element into ALL replicas from the same registers (no separate publish pass).
* ``reduce_to_owner`` / ``publish``: the unbucketed forms (one kernel per owned range, ordered by
  an epoch barrier on the symmetric flag pad), kept for runtimes that do not overlap.

No NCCL call moves bulk data.  The kernels are in ``csrc/peer_comm.cu``; the torch.distributed implementation
with identical semantics is ``owner_sharded.TorchComm``.
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, List, Tuple

import torch
import torch.distributed as dist

from ..ops import _cuda

_cuda.register("b200_peer_reduce_bf16", "peer_comm", "piillfs")
_cuda.register("b200_peer_publish", "peer_comm", "piills")
_cuda.register("b200_peer_barrier", "peer_comm", "piiipis")
_cuda.register("b200_peer_bucket_reduce", "peer_comm", "ppiiiiipifpiis")
_cuda.register("b200_peer_adamw", "peer_comm", "piilppppilfffffffppis")
_cuda.register("b200_peer_muon_update", "peer_comm", "piilpplfffpis")


def _ptr_array(ptrs: List[int]):
    arr = (ctypes.c_void_p * len(ptrs))(*ptrs)
    return arr


class PeerComm:
    supports_overlap = True
    PAD_WORDS = 16384       # [0, 64): barrier slots; then 32 words per flag block (16 ready + 16 acknowledgement flags)
    BUCKET_FLAG_BASE = 64
    BUCKET_FLAG_STRIDE = 32
    BARRIER_TIMEOUT_MS = 1800 * 1000  # default: the usual collective timeout of a training job

    def __init__(self, group, device: torch.device, barrier_timeout_ms: int = 0):
        if barrier_timeout_ms > 0:
            self.BARRIER_TIMEOUT_MS = int(barrier_timeout_ms)
        # the runtime keeps multicast (NVLS) objects out of the picture: plain peer loads/stores only
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem

        self._symm = symm_mem
        self.group = group if group is not None else dist.group.WORLD
        self.n = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.device = device
        self._handles: Dict[int, Tuple[torch.Tensor, object, object]] = {}
        self._epoch = 0
        pad = symm_mem.empty(self.PAD_WORDS, dtype=torch.int32, device=device)
        pad.zero_()
        self._pad = pad
        self._pad_hdl = symm_mem.rendezvous(pad, group=self.group)
        self._pad_ptrs = _ptr_array([int(p) for p in self._pad_hdl.buffer_ptrs])
        torch.cuda.synchronize(device)
        dist.barrier(group=self.group)

    def global_rank(self, r: int) -> int:
        return dist.get_global_rank(self.group, r)

    def allocate(self, numel: int, dtype, device) -> torch.Tensor:
        t = self._symm.empty(numel, dtype=dtype, device=device)
        t.zero_()
        # symmetric buffers bypass torch's caching allocator: memory reports add this counter
        self.allocated_bytes = getattr(self, "allocated_bytes", 0) + t.numel() * t.element_size()
        hdl = self._symm.rendezvous(t, group=self.group)
        self._handles[t.data_ptr()] = (t, hdl, _ptr_array([int(p) for p in hdl.buffer_ptrs]))
        return t

    def _peers(self, flat: torch.Tensor):
        return self._handles[flat.data_ptr()][2]

    def barrier(self) -> None:
        if self.n == 1:
            return
        self._epoch += 1
        st = _cuda.status_word(self.device)
        _cuda.call("b200_peer_barrier", ctypes.addressof(self._pad_ptrs), self.n, self.rank, self._epoch, st.data_ptr(),
                   self.BARRIER_TIMEOUT_MS, _cuda.stream())

    def bump(self, key) -> int:
        """Next value of the monotonic counter ``key``.  Flag values on the pad only ever grow, so every protocol
        that signals through the pad draws its epochs from here: a second runtime on the same communicator then
        continues where the first one stopped instead of meeting flags that already read "ready"."""
        c = self.__dict__.setdefault("_counters", {})
        c[key] = c.get(key, 0) + 1
        return c[key]

    @property
    def max_buckets(self) -> int:
        return (self.PAD_WORDS - self.BUCKET_FLAG_BASE) // self.BUCKET_FLAG_STRIDE

    def bucket_reduce(self, grad_flat: torch.Tensor, bucket: int, ranges, epoch: int, max_blocks: int = 0) -> None:
        """Signal that this rank's gradients of ``bucket`` are final, wait for the peers' signals of the same
        ``epoch`` and sum the owned ``ranges`` ((lo, hi) element pairs) over all ranks, in place.  Runs on the
        current stream; the caller puts it on a side stream that waits for the bucket's backward."""
        if self.n == 1:
            return
        if bucket >= self.max_buckets:
            raise ValueError(f"bucket {bucket} exceeds the flag pad ({self.max_buckets} buckets)")
        flat = [v for lo, hi in ranges if hi > lo for v in (lo, hi - lo)]
        arr = (ctypes.c_long * max(len(flat), 1))(*flat)
        st = _cuda.status_word(self.device)
        _cuda.call("b200_peer_bucket_reduce", ctypes.addressof(self._peers(grad_flat)), ctypes.addressof(self._pad_ptrs),
                   self.n, self.rank, int(grad_flat.dtype == torch.float32), self.BUCKET_FLAG_BASE + bucket * self.BUCKET_FLAG_STRIDE,
                   epoch & 0xFFFFFFFF, ctypes.addressof(arr), len(flat) // 2, 1.0, st.data_ptr(), self.BARRIER_TIMEOUT_MS,
                   int(max_blocks), _cuda.stream())

    def adamw_publish(self, param_flat, lo: int, p32, m, v, g, *, lr, beta1, beta2, eps, wd, step, gscale, skip,
                      max_blocks: int = 0) -> None:
        """AdamW on the owned slice ``[lo, lo + p32.numel())``; the new bf16 values go to every replica."""
        bc1, bc2 = 1.0 - beta1 ** step, 1.0 - beta2 ** step
        _cuda.call("b200_peer_adamw", ctypes.addressof(self._peers(param_flat)), self.n, self.rank, lo, p32.data_ptr(),
                   m.data_ptr(), v.data_ptr(), g.data_ptr(), int(g.dtype == torch.float32), p32.numel(), float(lr),
                   float(beta1), float(beta2), float(eps), float(wd), float(bc1), float(bc2), _cuda.ptr(gscale),
                   _cuda.ptr(skip), int(max_blocks), _cuda.stream())

    def muon_update_publish(self, param_flat, lo: int, p32, o, *, lr, wd, scale, skip, max_blocks: int = 0) -> None:
        """Muon update of one owned matrix at flat offset ``lo``; the new bf16 values go to every replica."""
        _cuda.call("b200_peer_muon_update", ctypes.addressof(self._peers(param_flat)), self.n, self.rank, lo, p32.data_ptr(),
                   o.data_ptr(), p32.numel(), float(lr), float(wd), float(scale), _cuda.ptr(skip), int(max_blocks),
                   _cuda.stream())

    def reduce_to_owner(self, grad_flat: torch.Tensor, ranges) -> None:
        if self.n == 1:
            return
        if grad_flat.dtype != torch.bfloat16:
            raise TypeError("the unbucketed peer reduce expects bf16 gradients")
        self.barrier()  # every rank has finished writing its gradients
        peers = self._peers(grad_flat)
        for lo, hi in ranges[self.rank]:
            if hi > lo:
                _cuda.call("b200_peer_reduce_bf16", ctypes.addressof(peers), self.n, self.rank, lo, hi - lo, 1.0, _cuda.stream())

    def publish_range(self, param_flat: torch.Tensor, lo: int, hi: int) -> None:
        """Store ``param_flat[lo:hi]`` into every other replica (no barrier)."""
        if self.n == 1 or hi <= lo:
            return
        es = param_flat.element_size()
        _cuda.call("b200_peer_publish", ctypes.addressof(self._peers(param_flat)), self.n, self.rank, lo * es, (hi - lo) * es,
                   _cuda.stream())

    def publish(self, param_flat: torch.Tensor, ranges) -> None:
        if self.n == 1:
            return
        for lo, hi in ranges[self.rank]:
            self.publish_range(param_flat, lo, hi)
        self.barrier()  # all replicas complete (and all peers are done reading my gradients)

    def broadcast_all(self, flat: torch.Tensor, src: int = 0) -> None:
        if self.n > 1:
            dist.broadcast(flat, src=self.global_rank(src), group=self.group)

    def all_reduce_sum(self, t: torch.Tensor) -> None:
        if self.n > 1:
            dist.all_reduce(t, group=self.group)
