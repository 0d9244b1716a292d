"""GEMMs that carry their collective: one tcgen05 kernel launch computes the tiles AND moves the
data between the GPUs of an NVSwitch domain over peer-mapped (symmetric) memory.

* ``ag_gemm``      all-gather of token rows  -> GEMM   (column-parallel projection, sequence-parallel TP)
* ``gemm_rs``      GEMM -> reduce-scatter of token rows (row-parallel projection; input gradient of the former)
* ``gemm_a2a``     GEMM -> all-to-all by head columns   (Ulysses: QKV projection straight into the head-sharded
                   layout; input gradient of the output projection)
* ``a2a_gemm``     all-to-all by head columns -> GEMM   (Ulysses: output projection; input gradient of QKV)

Every rank launches the same kernel with the same shapes.  Data moves with plain peer stores issued
by the kernel's own warps; per-buffer arrival counters in symmetric memory tell a consumer when a
source rank's block is complete, and all waits are bounded (a rank that gives up raises the status
word instead of spinning).  The kernels are in ``csrc/gemm_sm100.cu`` (``CommParams``).

The reference performs these steps as separate NCCL collectives around cuBLAS GEMMs
(src/lmms_engine/parallel/sequence_parallel/ulysses.py:101-330 for the all-to-alls, DTensor
``ColwiseParallel`` / ``RowwiseParallel`` in src/lmms_engine/parallel/qwen3_vl/parallelize.py:58-69).

With a group of one rank the same kernels run on ordinary device memory, which is how the
single-GPU numerics tests exercise them.
"""
from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from ..ops import _cuda

_cuda.register("b200_gemm_comm_bf16", "gemm_sm100", "pppiiiiiiifppps")
_cuda.register("b200_peer_memcpy", "peer_comm", "ppls")
_cuda.register("b200_peer_signal", "peer_comm", "pis")
_cuda.register("b200_peer_memcpy2d", "peer_comm", "plpllls")

_NVTX = os.environ.get("LMMS_B200_NVTX") == "1"
MAX_RANKS = 8
_FLAG_WORDS = 3 * MAX_RANKS
_ALIGN = 256


class SymmPool:
    """Bump allocator over symmetric-memory chunks (one rendezvous per chunk, not per buffer).
    All ranks must allocate in the same order, which any SPMD program does."""

    def __init__(self, group, device: torch.device, chunk_bytes: int = 256 << 20):
        self.group = group
        self.world = dist.get_world_size(group) if group is not None else 1
        self.rank = dist.get_rank(group) if group is not None else 0
        if self.world > MAX_RANKS:
            raise ValueError(f"fused collectives support at most {MAX_RANKS} ranks per group")
        self.device = device
        self.chunk_bytes = chunk_bytes
        self._chunks: List[Tuple[torch.Tensor, List[int]]] = []
        self._used = 0
        if self.world > 1:
            # plain peer loads / stores only: keep multicast objects out of the picture
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
            import torch.distributed._symmetric_memory as symm_mem

            self._symm = symm_mem

    def _new_chunk(self, nbytes: int) -> None:
        nbytes = max(self.chunk_bytes, (nbytes + _ALIGN - 1) // _ALIGN * _ALIGN)
        if self.world == 1:
            t = torch.zeros(nbytes, dtype=torch.uint8, device=self.device)
            ptrs = [t.data_ptr()]
        else:
            t = self._symm.empty(nbytes, dtype=torch.uint8, device=self.device)
            t.zero_()
            hdl = self._symm.rendezvous(t, group=self.group)
            ptrs = [int(p) for p in hdl.buffer_ptrs]
            self._hdl = getattr(self, "_hdl", []) + [hdl]
            # nobody may raise a flag in this chunk before every rank has zeroed it
            torch.cuda.synchronize(self.device)
            dist.barrier(group=self.group)
        self._chunks.append((t, ptrs))
        self._used = 0

    def alloc(self, nbytes: int) -> Tuple[torch.Tensor, List[int]]:
        nbytes = (nbytes + _ALIGN - 1) // _ALIGN * _ALIGN
        if not self._chunks or self._used + nbytes > self._chunks[-1][0].numel():
            self._new_chunk(nbytes)
        t, ptrs = self._chunks[-1]
        view = t[self._used:self._used + nbytes]
        out = (view, [p + self._used for p in ptrs])
        self._used += nbytes
        return out


class CommBuffer:
    """A bf16 region that every rank of the group can address, with its arrival counters.  ``t`` is
    the ``[rows, cols]`` matrix of the current call laid out at the start of the region."""

    def __init__(self, pool: SymmPool, capacity: int):
        raw, self.ptrs = pool.alloc(capacity * 2)
        self.raw = raw[: capacity * 2].view(torch.bfloat16)
        self.capacity = capacity
        self.t = self.raw.view(1, capacity)
        flag_raw, self.flag_ptrs = pool.alloc(_FLAG_WORDS * 4)
        self.flags = flag_raw[: _FLAG_WORDS * 4].view(torch.int32)
        self.n_in = 0    # arrive_in value reached by the calls made so far
        self.n_out = 0
        self.n_done = 0

    def shaped(self, rows: int, cols: int) -> "CommBuffer":
        self.t = self.raw[: rows * cols].view(rows, cols)
        return self


@dataclass
class HeadRoute:
    """Where every 64-column chunk of a [tokens, heads*dim] projection goes in the head-sharded
    layout ``[q heads of the rank | k heads | v heads]`` (device tables, one entry per chunk)."""

    chunk_dst: torch.Tensor
    chunk_col: torch.Tensor
    chunk_ndst: torch.Tensor
    cols_local: int
    kv_replicated: bool


def qkv_head_route(n_q: int, n_kv: int, head_dim: int, world: int, device) -> HeadRoute:
    """Routing of the fused QKV projection ``[q | k | v]`` for a group of ``world`` ranks.  Query
    heads must divide the group; KV heads either divide it or are replicated over ``world/n_kv``
    consecutive ranks (the reference repeats them the same way, ulysses.py:288-300)."""
    if head_dim % 64 or n_q % world or not (n_kv % world == 0 or world % n_kv == 0):
        raise ValueError(f"no fused route for {n_q} q / {n_kv} kv heads of {head_dim} over {world} ranks")
    hq_l = n_q // world
    rep = 1 if n_kv % world == 0 else world // n_kv
    hkv_l = max(n_kv // world, 1)
    cph = head_dim // 64
    dst, col, nd = [], [], []
    for h in range(n_q):
        for c in range(cph):
            dst.append(h // hq_l), col.append((h % hq_l) * head_dim + c * 64), nd.append(1)
    for part in range(2):  # k then v
        base = (hq_l + part * hkv_l) * head_dim
        for h in range(n_kv):
            for c in range(cph):
                if rep == 1:
                    dst.append(h // hkv_l), col.append(base + (h % hkv_l) * head_dim + c * 64), nd.append(1)
                else:
                    dst.append(h * rep), col.append(base + c * 64), nd.append(rep)
    mk = lambda v: torch.tensor(v, dtype=torch.int32, device=device)
    return HeadRoute(mk(dst), mk(col), mk(nd), (hq_l + 2 * hkv_l) * head_dim, rep > 1)


def out_head_route(n_q: int, head_dim: int, world: int, device) -> HeadRoute:
    """Routing of a ``[tokens, n_q*dim]`` matrix (gradient of the attention output) by query head."""
    if head_dim % 64 or n_q % world:
        raise ValueError("no fused route")
    hq_l = n_q // world
    cph = head_dim // 64
    dst = [h // hq_l for h in range(n_q) for _ in range(cph)]
    col = [(h % hq_l) * head_dim + c * 64 for h in range(n_q) for c in range(cph)]
    mk = lambda v: torch.tensor(v, dtype=torch.int32, device=device)
    return HeadRoute(mk(dst), mk(col), mk([1] * len(dst)), hq_l * head_dim, False)


def _mat_ok(t: torch.Tensor) -> bool:
    return t.is_cuda and t.dtype == torch.bfloat16 and t.dim() == 2 and t.stride(1) == 1 and t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0


class FusedComm:
    """Per-group context: symmetric pool, named buffers, launch bookkeeping."""

    def __init__(self, group, device: torch.device, wait_ms: int = 60000, chunk_bytes: int = 256 << 20):
        self.pool = SymmPool(group, device, chunk_bytes)
        self.group, self.world, self.rank, self.device = group, self.pool.world, self.pool.rank, device
        self.wait_ms = wait_ms
        self._buffers: Dict[Tuple, CommBuffer] = {}
        self._turn: Dict = {}
        self.max_ctas = 0
        self.launches = 0
        self.push_ctas: Optional[int] = None  # None: chosen per call from the copy volume; 0: push from every CTA
        self.ag_engine: Optional[str] = None  # force "sm" or "ce" for the all-gather copy
        self.a2a_engine: Optional[str] = None  # likewise for the column-block exchange of a2a_gemm
        # GEMM -> reduce-scatter with the scattering epilogue beat GEMM + NCCL on 2 and 4 ranks (1.22x, 1.11x)
        # and lost on 8 (0.86x: peer stores from the epilogue warps reach ~230 GB/s there)
        self.rs_fused_max_world = 4
        self._side: Optional[torch.cuda.Stream] = None
        self.trace: Optional[torch.Tensor] = None  # set to an int64[6] device tensor to record a launch timeline

    def buffer(self, key, rows: int, cols: int, rotate: bool = False) -> CommBuffer:
        """The named buffer, shaped for this call.  It is re-created (rows rounded up to 1024) only
        when a call needs more room than any earlier one, identically on every rank.

        ``rotate`` alternates between two buffers of that name.  A gather buffer that the next call
        with the same name overwrites needs it: a rank can start call n+2 only after call n+1, in
        which it waited for every other rank's block, and a rank sends its block of call n+1 only
        after everything it queued behind call n (the readers of that buffer) has finished; so the
        buffer of call n is free on every rank when call n+2 writes it, without a handshake."""
        if rotate:
            turn = self._turn[key] = self._turn.get(key, 0) ^ 1
            key = (key, "turn", turn)
        b = self._buffers.get(key)
        if b is None or b.capacity < rows * cols:
            b = self._buffers[key] = CommBuffer(self.pool, ((rows + 1023) // 1024 * 1024) * cols)
        return b.shaped(rows, cols)

    # ------------------------------------------------------------------ launch
    def _launch(self, a, b, c, M, N, K, b_mn, alpha, bias, *, push=None, wait_mode=0, rows_per_src=0, k_per_src=0,
                kb_src=None, m_rot=0, k_rot=0, scatter=None, own_direct=False, push_ctas=0):
        ca = (ctypes.c_longlong * 96)()
        ca[0], ca[1], ca[2] = self.rank, self.world, self.wait_ms
        if push is not None:
            buf: CommBuffer = push["buf"]
            ca[3] = 0 if push.get("external") else 1
            ca[80] = 1 if push.get("external") else 0
            ca[6] = push["block_rows"]
            ca[7] = buf.t.stride(0)
            ca[8] = push["dst_off"]
            ca[9] = push["rows"]
            segs = push["segs"]  # (src tensor, dst col, cols)
            ca[10] = len(segs)
            for i, (src, dcol, cols) in enumerate(segs):
                if not _mat_ok(src):
                    raise TypeError("pushed blocks must be 2-D bf16 CUDA matrices with unit inner stride")
                ca[11 + i], ca[14 + i], ca[17 + i], ca[73 + i] = src.data_ptr(), dcol, cols, src.stride(0)
            ca[20] = buf.n_in
            ca[21] = 1 if push.get("handshake", False) else 0
            ca[22] = buf.n_done
            for r in range(self.world):
                ca[24 + r], ca[32 + r] = buf.ptrs[r], buf.flag_ptrs[r]
        if kb_src is not None:
            ca[4] = kb_src.data_ptr()
        ca[40], ca[41], ca[42], ca[43], ca[44] = wait_mode, rows_per_src, k_per_src, m_rot, k_rot
        if scatter is not None:
            sb: CommBuffer = scatter["buf"]
            ca[45] = scatter["mode"]
            ca[46] = sb.t.stride(0)
            ca[47] = scatter.get("slot_stride", 0)
            route: Optional[HeadRoute] = scatter.get("route")
            if route is not None:
                ca[48], ca[49], ca[50] = route.chunk_dst.data_ptr(), route.chunk_col.data_ptr(), route.chunk_ndst.data_ptr()
            ca[51] = scatter.get("row_off", 0)
            ca[52] = sb.n_out
            ca[53] = sb.n_done
            out = scatter.get("reduce_out")
            if out is not None:
                ca[54], ca[55] = out.data_ptr(), out.stride(0)
            for r in range(self.world):
                ca[56 + r], ca[64 + r] = sb.ptrs[r], sb.flag_ptrs[r]
        ca[72] = self.max_ctas
        ca[76] = 1 if own_direct else 0
        push_ctas = min(int(push_ctas), 64) if (push is not None and wait_mode != 2 and not push.get("external")) else 0
        ca[78] = push_ctas
        # peer stores are limited per SM, so the copy is spread over all CTAs; the epilogue warps join it
        # only where no tile can complete before the blocks have landed (every tile needs every source)
        ca[79] = 1 if wait_mode == 2 else 0
        if self.trace is not None:  # CTA 0's timeline of this launch, six globaltimer stamps
            ca[77] = self.trace.data_ptr()
        st = _cuda.status_word(self.device)
        if _NVTX:
            torch.cuda.nvtx.range_push(f"fused_gemm M{M} N{N} K{K} push{int(push is not None)} wait{wait_mode} scatter{scatter['mode'] if scatter else 0}")
        ctas = _cuda.call_raw(
            "b200_gemm_comm_bf16", a.data_ptr(), b.data_ptr(), c.data_ptr() if c is not None else 0, M, N, K,
            a.stride(0), b.stride(0), c.stride(0) if c is not None else 0, int(b_mn), float(alpha), _cuda.ptr(bias),
            ctypes.addressof(ca), st.data_ptr(), _cuda.stream(),
        )
        if _NVTX:
            torch.cuda.nvtx.range_pop()
        if ctas <= 0:
            raise RuntimeError(f"b200_gemm_comm_bf16 refused the launch (code {ctas}) for M={M} N={N} K={K}")
        if push is not None and push.get("external"):
            push["buf"].n_in += 1
        elif push is not None:
            push["buf"].n_in += push_ctas if push_ctas > 0 else ctas
            if ca[21]:
                push["buf"].n_done += push_ctas if push_ctas > 0 else ctas
        if scatter is not None:
            if scatter["mode"] == 1:
                # one count per epilogue warp and tile that a rank sends to another
                scatter["buf"].n_out += 4 * (rows_per_src // 128) * ((N + 255) // 256)
                scatter["buf"].n_done += ctas
            else:
                scatter["buf"].n_out += ctas - push_ctas
        self.launches += 1
        return ctas

    def _push_ctas(self, push_bytes: float, flops: float) -> int:
        """Dedicated copy CTAs are off by default: measured peer-store throughput is a few GB/s per SM
        whatever the thread count, so a copy confined to a few SMs is slower than one spread over all."""
        return 0

    @staticmethod
    def _bshape(w: torch.Tensor, b_mn: bool) -> Tuple[int, int]:
        return (w.shape[1], w.shape[0]) if b_mn else (w.shape[0], w.shape[1])  # (N, K)

    # ------------------------------------------------------------------ all-gather rows -> GEMM
    def ag_gemm(self, x: torch.Tensor, w: torch.Tensor, bias=None, b_mn: bool = False, key="ag", engine: Optional[str] = None):
        """``y = concat_r(x_r) @ op(w)^T (+ bias)``; returns ``(y, gathered)`` where ``gathered`` is the
        shared gather buffer (valid until the second next call with the same key).

        ``engine="ce"``: the copy engines move this rank's rows into the peers' buffers on a side
        stream (one device-to-device copy and one flag per peer) while the kernel computes the rows
        it already has and waits, tile by tile, for the flags.  ``engine="sm"``: two warps of every
        CTA store the rows themselves.  Default: ``ce`` for more than two ranks - stores issued next
        to a running main loop reach only about 150 GB/s, which hides one peer's block but not more."""
        Ms, K = x.shape
        N, Kw = self._bshape(w, b_mn)
        if K != Kw or Ms % 128:
            raise ValueError("ag_gemm needs matching K and a multiple of 128 rows per rank")
        if engine is None:
            engine = self.ag_engine or ("ce" if self.world > 2 else "sm")
        buf = self.buffer(key, Ms * self.world, K, rotate=True)
        y = torch.empty((Ms * self.world, N), dtype=torch.bfloat16, device=x.device)
        push = dict(buf=buf, block_rows=0, dst_off=self.rank * Ms * buf.t.stride(0), rows=Ms, segs=[(x, 0, K)])
        if engine == "ce" and self.world > 1:
            x = x if x.is_contiguous() else x.contiguous()
            push["segs"] = [(x, 0, K)]
            push["external"] = True
            main = torch.cuda.current_stream()
            if self._side is None:
                self._side = torch.cuda.Stream(device=self.device)
            ready = torch.cuda.Event()
            ready.record(main)
            self._side.wait_event(ready)
            nbytes, off = Ms * K * 2, self.rank * Ms * K * 2
            for d in range(self.world):
                r = (self.rank - 1 - d) % self.world  # the order in which the ranks need this block; own copy last
                _cuda.call("b200_peer_memcpy", buf.ptrs[r] + off, x.data_ptr(), nbytes, self._side.cuda_stream)
                flag = (ctypes.c_void_p * 1)(buf.flag_ptrs[r] + 4 * self.rank)
                _cuda.call("b200_peer_signal", ctypes.addressof(flag), 1, self._side.cuda_stream)
            done = torch.cuda.Event()
            done.record(self._side)
        self._launch(buf.t, w, y, Ms * self.world, N, K, b_mn, 1.0, bias, push=push, wait_mode=1, rows_per_src=Ms,
                     m_rot=self.rank * (Ms // 128), own_direct=True)
        if push.get("external"):
            torch.cuda.current_stream().wait_event(done)  # x and the buffer stay valid for what follows
        return y, buf.t

    # ------------------------------------------------------------------ GEMM -> reduce-scatter rows
    def gemm_rs(self, x: torch.Tensor, w: torch.Tensor, b_mn: bool = False, key="rs", regather=None):
        """``y_r = sum_ranks (x @ op(w)^T)[rows of r]``.  ``regather=(x_local, key)`` additionally
        all-gathers ``x_local`` into the buffer of that key while the tiles run (the weight
        gradient of a column-parallel layer needs the gathered input again) and returns it."""
        M, K = x.shape
        N, Kw = self._bshape(w, b_mn)
        if K != Kw or M % (128 * self.world) or N % 8:
            raise ValueError("gemm_rs needs matching K and rows that split into 128-row blocks per rank")
        Ms = M // self.world
        slots = self.buffer(key, self.world * Ms, N)
        out = torch.empty((Ms, N), dtype=torch.bfloat16, device=x.device)
        scatter = dict(buf=slots, mode=1, slot_stride=Ms * slots.t.stride(0), reduce_out=out)
        push, gathered = None, None
        if regather is not None:
            xl, gkey = regather
            gb = self.buffer(gkey, xl.shape[0] * self.world, xl.shape[1], rotate=True)
            push = dict(buf=gb, block_rows=0, dst_off=self.rank * xl.shape[0] * gb.t.stride(0), rows=xl.shape[0],
                        segs=[(xl, 0, xl.shape[1])])
            gathered = gb.t
        pc = 0
        if push is not None:
            pc = self.push_ctas if self.push_ctas is not None else self._push_ctas(push["rows"] * push["segs"][0][2] * 2.0 * self.world, 2.0 * M * N * K)
        self._launch(x, w, None, M, N, K, b_mn, 1.0, None, push=push, rows_per_src=Ms,
                     m_rot=((self.rank + 1) % self.world) * (Ms // 128), scatter=scatter, push_ctas=pc)
        return (out, gathered) if regather is not None else out

    # ------------------------------------------------------------------ GEMM -> all-to-all by heads
    def gemm_a2a(self, x: torch.Tensor, w: torch.Tensor, route: HeadRoute, bias=None, b_mn: bool = False, key="qkv"):
        """``(x @ op(w)^T + bias)`` with column chunk ``c`` of my ``Tl`` rows stored at rows
        ``[rank*Tl, (rank+1)*Tl)`` of rank ``route.chunk_dst[c]``'s ``[world*Tl, cols_local]`` buffer.
        The buffer of ``key`` persists (the caller keeps it for its backward pass)."""
        Tl, K = x.shape
        N, Kw = self._bshape(w, b_mn)
        if K != Kw or N != route.chunk_dst.numel() * 64:
            raise ValueError("route does not match the projection")
        dst = self.buffer(key, Tl * self.world, route.cols_local)
        scatter = dict(buf=dst, mode=2, route=route, row_off=self.rank * Tl)
        self._launch(x, w, None, Tl, N, K, b_mn, 1.0, bias, scatter=scatter)
        return dst.t

    # ------------------------------------------------------------------ all-to-all by heads -> GEMM
    def a2a_gemm(self, parts: Sequence[Tuple[torch.Tensor, int]], w: torch.Tensor, cols_total: int, kb_src=None,
                 b_mn: bool = False, bias=None, key="o", k_rot: int = 0, rotate: bool = True, engine: Optional[str] = None):
        """``parts`` = ``[(src [world*Tl, c_i], dst_col_i), ...]``: rows ``[r*Tl, (r+1)*Tl)`` of every
        source go to rank r at columns ``dst_col_i``; then ``y = gathered[Tl, cols_total] @ op(w)^T``.
        Returns ``(y, gathered)``; ``gathered`` is the shared buffer of ``key``."""
        T = parts[0][0].shape[0]
        Tl = T // self.world
        N, Kw = self._bshape(w, b_mn)
        if Kw != cols_total:
            raise ValueError("weight does not match the gathered width")
        buf = self.buffer(key, Tl, cols_total, rotate=rotate)
        y = torch.empty((Tl, N), dtype=torch.bfloat16, device=w.device)
        segs = [(src, dcol, src.shape[1]) for src, dcol in parts]
        push = dict(buf=buf, block_rows=Tl, dst_off=0, rows=Tl, segs=segs)
        kps = cols_total // self.world
        # a single source whose block sits at my rank's column range can be read in place
        direct = len(parts) == 1 and kb_src is None and parts[0][1] == self.rank * kps and parts[0][0].shape[1] == kps
        engine = engine or self.a2a_engine or ("ce" if self.world > 2 else "sm")
        if engine == "ce" and self.world > 1:
            # copy engines move the column blocks (pitched copies) on a side stream; one flag per peer
            push["external"] = True
            main = torch.cuda.current_stream()
            if self._side is None:
                self._side = torch.cuda.Stream(device=self.device)
            ready = torch.cuda.Event()
            ready.record(main)
            self._side.wait_event(ready)
            for d in range(self.world):
                r = (self.rank - 1 - d) % self.world if direct else (self.rank - d) % self.world
                for src, dcol, cols in segs:
                    if not _mat_ok(src):
                        raise TypeError("a2a_gemm sources must be 2-D bf16 CUDA matrices with unit inner stride")
                    _cuda.call("b200_peer_memcpy2d", buf.ptrs[r] + dcol * 2, cols_total * 2,
                               src.data_ptr() + r * Tl * src.stride(0) * 2, src.stride(0) * 2, cols * 2, Tl, self._side.cuda_stream)
                flag = (ctypes.c_void_p * 1)(buf.flag_ptrs[r] + 4 * self.rank)
                _cuda.call("b200_peer_signal", ctypes.addressof(flag), 1, self._side.cuda_stream)
            done = torch.cuda.Event()
            done.record(self._side)
        self._launch(buf.t, w, y, Tl, N, cols_total, b_mn, 1.0, bias, push=push, wait_mode=2, k_per_src=kps,
                     kb_src=kb_src, k_rot=k_rot, own_direct=direct)
        if push.get("external"):
            torch.cuda.current_stream().wait_event(done)
        return y, buf.t


def qkv_kb_sources(n_q: int, n_kv: int, head_dim: int, world: int, device) -> torch.Tensor:
    """Source rank of every 64-wide k-block of the global ``[q | k | v]`` column order."""
    hq_l, hkv_l = n_q // world, n_kv // world
    cph = head_dim // 64
    src = [h // hq_l for h in range(n_q) for _ in range(cph)]
    for _ in range(2):
        src += [h // hkv_l for h in range(n_kv) for _ in range(cph)]
    return torch.tensor(src, dtype=torch.int32, device=device)
