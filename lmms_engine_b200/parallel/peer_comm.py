"""Peer-memory implementation of the owner-sharded runtime's collective steps.

The flat parameter and gradient buffers are allocated from torch's symmetric-memory pool and
mapped into every rank of the group (NVLink / NVSwitch).  ``reduce_to_owner`` is then one
kernel per owned range that PULLS the range from all peers and sums it in fp32;
``publish`` is one kernel per owned range that PUSHES the updated bf16 values into every
replica; an epoch barrier on a symmetric flag pad orders the phases.  No NCCL call moves
bulk data.  The kernels are in ``csrc/peer_comm.cu``; the torch.distributed implementation
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


def _ptr_array(ptrs: List[int]):
    arr = (ctypes.c_void_p * len(ptrs))(*ptrs)
    return arr


class PeerComm:
    BARRIER_TIMEOUT_MS = 20000

    def __init__(self, group, device: torch.device):
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
        pad = symm_mem.empty(1024, dtype=torch.int32, device=device)
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

    def reduce_to_owner(self, grad_flat: torch.Tensor, ranges) -> None:
        if self.n == 1:
            return
        if grad_flat.dtype != torch.bfloat16:
            raise TypeError("peer reduce expects bf16 gradients")
        self.barrier()  # every rank has finished writing its gradients
        peers = self._peers(grad_flat)
        for lo, hi in ranges[self.rank]:
            if hi > lo:
                _cuda.call("b200_peer_reduce_bf16", ctypes.addressof(peers), self.n, self.rank, lo, hi - lo, 1.0, _cuda.stream())

    def publish(self, param_flat: torch.Tensor, ranges) -> None:
        if self.n == 1:
            return
        peers = self._peers(param_flat)
        es = param_flat.element_size()
        for lo, hi in ranges[self.rank]:
            if hi > lo:
                _cuda.call("b200_peer_publish", ctypes.addressof(peers), self.n, self.rank, lo * es, (hi - lo) * es, _cuda.stream())
        self.barrier()  # all replicas complete (and all peers are done reading my gradients)

    def broadcast_all(self, flat: torch.Tensor, src: int = 0) -> None:
        if self.n > 1:
            dist.broadcast(flat, src=self.global_rank(src), group=self.group)

    def all_reduce_sum(self, t: torch.Tensor) -> None:
        if self.n > 1:
            dist.all_reduce(t, group=self.group)
