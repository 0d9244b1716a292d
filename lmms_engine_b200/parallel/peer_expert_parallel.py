"""Expert parallelism over peer memory: the dispatch and combine all-to-alls are row-mapped peer
copies issued by this GPU's own kernels (``csrc/ep_comm.cu``).

Per layer:

1. the count matrix is all-gathered and read on the host once (like the reference,
   src/lmms_engine/parallel/expert_parallel/utils.py:11-77) to size the expert-major layout of every
   rank; from it every local row gets its destination ``(rank, row)``.  With ``LMMS_B200_EP_DEVICE_LAYOUT=1`` the
   same layout is computed on the device for receive areas of a fixed capacity, and nothing is read back;
2. **push**: one kernel gathers token rows through the local permutation and stores them directly at
   their final expert-major row on the owning rank (no send buffer, no receive-side regroup);
3. grouped tcgen05 GEMMs on the owner (``ops.moe.grouped_mlp``);
4. **pull**: one kernel reads each token's ``k`` expert outputs from the owners' buffers, applies the
   router weights and sums (combine all-to-all + weighted scatter-add in one pass).

Backward mirrors it: the gradient of the combine is a push (with the router weight as a per-row
scalar) plus a scalar pull for the router-weight gradients; the gradient of the dispatch is a pull
with unit weights.  Staging buffers live in the group's symmetric pool and are sized from the count
matrix; safety of their reuse follows from the alternation of pushes and pulls (a push ends with
every rank's arrival, a pull starts with every rank's readiness).
"""
from __future__ import annotations

import ctypes
import os
from typing import List, Optional

import torch
import torch.distributed as dist

from ..ops import _cuda
from ..ops import moe as moe_ops
from .expert_parallel import ExpertParallel, _pad
from .fused_comm import SymmPool

TILE = moe_ops.TILE

_cuda.register("b200_ep_push", "ep_comm", "plpppplilpppiiippills")
_cuda.register("b200_ep_pull", "ep_comm", "plppppliilppiiipills")
_cuda.register("b200_ep_pull_scalar", "ep_comm", "pppplpppiiipills")


def _ptrs(v: List[int]):
    return (ctypes.c_void_p * len(v))(*v)


class _Stage:
    """One symmetric staging area: ``cap`` rows of ``H`` bf16 plus two fp32 scalars per row."""

    def __init__(self, pool: SymmPool, cap: int, H: int):
        self.cap, self.H = cap, H
        raw, self.ptrs = pool.alloc(cap * H * 2)
        self.t = raw[: cap * H * 2].view(torch.bfloat16).view(cap, H)
        s_raw, self.s_ptrs = pool.alloc(cap * 4)
        self.s = s_raw[: cap * 4].view(torch.float32)
        self.c_ptrs, self.c_sptrs = _ptrs(self.ptrs), _ptrs(self.s_ptrs)


class PeerExpertParallel(ExpertParallel):
    WAIT_MS = 60000

    def __init__(self, group, num_experts: int, device: torch.device):
        super().__init__(group, num_experts)
        self.device = device
        self.pool = SymmPool(group, device)
        flag_raw, flag_ptrs = self.pool.alloc(4 * 16 * 4)
        self.flags = flag_raw[:256].view(torch.int32)
        self.c_flags = _ptrs(flag_ptrs)
        self.counter = torch.zeros(1, dtype=torch.int32, device=device)
        self.push_epoch = self.pull_epoch = self.scalar_epoch = 0
        self.x_stage: Optional[_Stage] = None  # peers push into it
        self.y_stage: Optional[_Stage] = None  # peers pull from it
        self.launches = 0
        # LMMS_B200_EP_DEVICE_LAYOUT=1: no host read of the count matrix per layer (fixed-capacity receive areas,
        # overflow reported through the status word); costs activation memory in proportion to the capacity factor
        self.device_layout = os.environ.get("LMMS_B200_EP_DEVICE_LAYOUT", "0") == "1"
        self.capacity_factor = float(os.environ.get("LMMS_B200_EP_CAPACITY", "1.5"))

    # ------------------------------------------------------------------ layout
    def _stages(self, rows_needed: int, H: int):
        if self.x_stage is None or self.x_stage.cap < rows_needed or self.x_stage.H != H:
            cap = (rows_needed + 4095) // 4096 * 4096
            self.x_stage = _Stage(self.pool, cap, H)
            self.y_stage = _Stage(self.pool, cap, H)
        return self.x_stage, self.y_stage

    def layout(self, counts: torch.Tensor, perm: moe_ops.Permutation):
        """Destination ``(rank, row)`` of every local row, my own expert-major layout, and the row
        capacity that every rank needs (identical on all ranks)."""
        all_counts = torch.empty(self.ep * self.E, dtype=counts.dtype, device=counts.device)
        dist.all_gather_into_tensor(all_counts, counts.contiguous(), group=self.group)
        C = all_counts.view(self.ep, self.E).cpu()
        P = (C + TILE - 1) // TILE * TILE  # padded segment sizes, [source, expert]
        El, me = self.El, self.rank
        # owner r lays out expert e as [source 0 | source 1 | ...]; experts in order
        per_expert = P.sum(0)  # rows of expert e on its owner
        start_on_owner = torch.zeros(self.E, dtype=torch.long)
        for r in range(self.ep):
            seg = per_expert[r * El:(r + 1) * El]
            start_on_owner[r * El:(r + 1) * El] = torch.cumsum(seg, 0) - seg
        before_me = P[:me].sum(0)  # rows of earlier sources inside expert e's block
        send_base = (start_on_owner + before_me).to(torch.int32).to(counts.device)
        rows_per_rank = per_expert.view(self.ep, El).sum(1)
        dev = counts.device
        # expert of every local row (local layout is by global expert id, padded per expert)
        e_row = perm.tile_expert.long().repeat_interleave(TILE)
        live = e_row >= 0
        e_safe = e_row.clamp(min=0)
        pos = torch.arange(e_row.numel(), device=dev) - perm.expert_start.long()[e_safe]
        dest_row = torch.where(live, send_base.long()[e_safe] + pos, torch.zeros_like(pos)).to(torch.int32)
        dest_rank = torch.where(live, e_safe // El, torch.full_like(e_safe, -1)).to(torch.int32)
        my_rows = int(rows_per_rank[me])
        mine = per_expert[me * El:(me + 1) * El]
        expert_start = torch.zeros(El + 1, dtype=torch.int32)
        expert_start[1:] = torch.cumsum(mine, 0).to(torch.int32)
        tile_expert = torch.repeat_interleave(torch.arange(El, dtype=torch.int32), (mine // TILE)).to(dev)
        local = moe_ops.Permutation(row_of=None, token_of_row=None, weight_of_row=None, tile_expert=tile_expert,
                                    expert_start=expert_start.to(dev), rows=my_rows, n_experts=El)
        return dest_rank, dest_row, local, int(rows_per_rank.max())

    def capacity(self, T: int, k: int) -> int:
        """Rows reserved per rank when the layout is computed on the device: ``capacity_factor`` x the balanced share
        (``T * k`` rows when every rank brings ``T`` tokens) plus the worst-case tile padding."""
        rows = int(self.capacity_factor * T * k) + self.ep * self.El * TILE
        return (rows + 4095) // 4096 * 4096

    def layout_device(self, counts: torch.Tensor, perm: moe_ops.Permutation, cap: int):
        """``layout`` without the host: the same destinations and expert-major layout as tensors computed on the device
        from the gathered count matrix, for a receive area of ``cap`` rows known before the counts are.  Rows that would
        land beyond ``cap`` are not sent (destination rank -1) and raise the overflow status word, which the next status
        check turns into an exception: raise ``capacity_factor`` (or use the host layout) for such routing."""
        all_counts = torch.empty(self.ep * self.E, dtype=counts.dtype, device=counts.device)
        dist.all_gather_into_tensor(all_counts, counts.contiguous(), group=self.group)
        return self.layout_from_counts(all_counts.view(self.ep, self.E), perm, cap, self.rank, self.El,
                                       _cuda.status_word(self.device) if counts.is_cuda else None)

    @staticmethod
    def layout_from_counts(C: torch.Tensor, perm: moe_ops.Permutation, cap: int, me: int, El: int, status: Optional[torch.Tensor] = None):
        ep, E = C.shape
        dev = C.device
        P = (C.long() + TILE - 1) // TILE * TILE             # padded segment sizes, [source, expert]
        per_expert = P.sum(0)                                # rows of expert e on its owner
        seg = per_expert.view(ep, El)
        start_on_owner = (seg.cumsum(1) - seg).flatten()     # owner lays out expert e as [source 0 | source 1 | ...]
        before_me = P[:me].sum(0)
        send_base = start_on_owner + before_me
        e_row = perm.tile_expert.long().repeat_interleave(TILE)
        live = e_row >= 0
        e_safe = e_row.clamp(min=0)
        pos = torch.arange(e_row.numel(), device=dev) - perm.expert_start.long()[e_safe]
        dest_row = torch.where(live, send_base[e_safe] + pos, torch.zeros_like(pos))
        fits = dest_row < cap
        dest_rank = torch.where(live & fits, e_safe // El, torch.full_like(e_safe, -1)).to(torch.int32)
        dest_row = torch.where(fits, dest_row, torch.zeros_like(dest_row)).to(torch.int32)
        if status is not None:  # any rank's area too small: every rank learns of it from the same count matrix
            over = (seg.sum(1) > cap).any()
            status.copy_(torch.where(over, torch.full_like(status, 4), status))
        mine = per_expert[me * El:(me + 1) * El]
        expert_start = torch.cat([mine.new_zeros(1), mine.cumsum(0)]).clamp(max=cap).to(torch.int32)
        tile_row = torch.arange(cap // TILE, device=dev) * TILE
        tile_expert = torch.searchsorted(expert_start[1:].long(), tile_row, right=True)
        tile_expert = torch.where(tile_row < expert_start[-1].long(), tile_expert, torch.full_like(tile_expert, -1)).to(torch.int32)
        local = moe_ops.Permutation(row_of=None, token_of_row=None, weight_of_row=None, tile_expert=tile_expert,
                                    expert_start=expert_start, rows=cap, n_experts=El)
        return dest_rank, dest_row, local, cap

    # ------------------------------------------------------------------ kernels
    def push(self, x, perm, dest_rank, dest_row, scalar=None):
        self.push_epoch += 1
        st = _cuda.status_word(self.device)
        xs = self.x_stage
        _cuda.call("b200_ep_push", x.data_ptr(), x.stride(0), perm.token_of_row.data_ptr(), _cuda.ptr(scalar),
                   dest_rank.data_ptr(), dest_row.data_ptr(), dest_rank.numel(), x.shape[1], xs.t.stride(0),
                   ctypes.addressof(xs.c_ptrs), ctypes.addressof(xs.c_sptrs), ctypes.addressof(self.c_flags), self.ep,
                   self.rank, self.push_epoch, self.counter.data_ptr(), st.data_ptr(), self.WAIT_MS, x.shape[0], xs.cap,
                   _cuda.stream())
        self.launches += 1

    def pull(self, stage: _Stage, row_of, w, dest_rank, dest_row, T: int, k: int, dtype):
        self.pull_epoch += 1
        out = torch.empty((T, stage.H), dtype=dtype, device=self.device)
        st = _cuda.status_word(self.device)
        _cuda.call("b200_ep_pull", out.data_ptr(), out.stride(0), row_of.data_ptr(), _cuda.ptr(w), dest_rank.data_ptr(),
                   dest_row.data_ptr(), T, k, stage.H, stage.t.stride(0), ctypes.addressof(stage.c_ptrs),
                   ctypes.addressof(self.c_flags), self.ep, self.rank, self.pull_epoch, st.data_ptr(), self.WAIT_MS,
                   dest_rank.numel(), stage.cap, _cuda.stream())
        self.launches += 1
        return out

    def pull_scalar(self, stage: _Stage, row_of, dest_rank, dest_row):
        self.scalar_epoch += 1
        out = torch.empty(row_of.shape, dtype=torch.float32, device=self.device)
        st = _cuda.status_word(self.device)
        _cuda.call("b200_ep_pull_scalar", out.data_ptr(), row_of.data_ptr(), dest_rank.data_ptr(), dest_row.data_ptr(),
                   row_of.numel(), ctypes.addressof(stage.c_ptrs), ctypes.addressof(stage.c_sptrs),
                   ctypes.addressof(self.c_flags), self.ep, self.rank, self.scalar_epoch, st.data_ptr(), self.WAIT_MS,
                   dest_rank.numel(), stage.cap, _cuda.stream())
        self.launches += 1
        return out

    # ------------------------------------------------------------------ layer
    def __call__(self, x, idx, w, counts, experts) -> torch.Tensor:
        perm = moe_ops.build_permutation(idx, w, counts)  # by global expert id
        if self.device_layout:
            dest_rank, dest_row, local, cap = self.layout_device(counts, perm, self.capacity(*idx.shape))
        else:
            dest_rank, dest_row, local, cap = self.layout(counts, perm)
        self._stages(cap, x.shape[1])
        grouped = _PeerDispatch.apply(x.contiguous(), self, perm, dest_rank, dest_row, local.rows)
        yp = experts(grouped, local)
        return _PeerCombine.apply(yp, w, self, perm, dest_rank, dest_row)


class _PeerDispatch(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, ep: PeerExpertParallel, perm, dest_rank, dest_row, my_rows):
        ep.push(x, perm, dest_rank, dest_row)
        ctx.ep, ctx.maps, ctx.shape = ep, (perm.row_of, dest_rank, dest_row), x.shape
        return ep.x_stage.t[:my_rows].clone()  # own copy: the staging area is reused by the next push

    @staticmethod
    def backward(ctx, dg):
        ep = ctx.ep
        row_of, dest_rank, dest_row = ctx.maps
        T, H = ctx.shape
        ep.y_stage.t[: dg.shape[0]].copy_(dg)
        dx = ep.pull(ep.y_stage, row_of, None, dest_rank, dest_row, T, row_of.shape[1], dg.dtype)
        return dx, None, None, None, None, None


class _PeerCombine(torch.autograd.Function):
    @staticmethod
    def forward(ctx, yp, w, ep: PeerExpertParallel, perm, dest_rank, dest_row):
        ep.y_stage.t[: yp.shape[0]].copy_(yp)
        wf = w.detach().float().contiguous()
        T, k = w.shape
        out = ep.pull(ep.y_stage, perm.row_of, wf, dest_rank, dest_row, T, k, yp.dtype)
        ctx.ep, ctx.perm, ctx.maps = ep, perm, (dest_rank, dest_row)
        ctx.save_for_backward(yp, w)
        return out

    @staticmethod
    def backward(ctx, dout):
        yp, w = ctx.saved_tensors
        ep, perm = ctx.ep, ctx.perm
        dest_rank, dest_row = ctx.maps
        rows = yp.shape[0]
        # gradient rows travel to the experts together with the router weight of their slot
        ep.push(dout.contiguous(), perm, dest_rank, dest_row, scalar=perm.weight_of_row)
        g = ep.x_stage.t[:rows]
        wrow = ep.x_stage.s[:rows]
        d_yp = moe_ops.row_scale_dot(g, yp, wrow, ep.y_stage.s[:rows])
        dw = ep.pull_scalar(ep.y_stage, perm.row_of, dest_rank, dest_row).to(w.dtype)
        return d_yp, dw, None, None, None, None
