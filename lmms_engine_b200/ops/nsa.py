"""Native sparse attention over packed documents: three causal branches mixed by per-head sigmoid gates.

* **compressed**: keys / values pooled over windows of ``kernel_size`` tokens every ``kernel_stride``
  tokens (average, learned per-position weights, or a learned linear map of the flattened window, keys
  with a learned intra-window position term); a query sees a window once the window has ended;
* **selected**: the compressed branch's probabilities, summed over the query heads of a KV group and
  spread onto selection blocks of ``block_size`` tokens by overlap, pick ``topk`` blocks per query and KV
  head (the first ``init_blocks`` and the last ``local_blocks`` always); the query attends causally to the
  tokens of its blocks;
* **sliding**: causal attention over the last ``window_size`` tokens (the varlen tcgen05 kernel).

Same call structure as the patched attention of src/lmms_engine/models/bagel/nsa_op.py:25-159, which
drives an external Triton package; this file states the arithmetic in PyTorch.  The selected branch gathers the
chosen blocks per query chunk when the document is long (work proportional to ``topk * block_size``) and runs as
masked attention when it is short; no gradient flows through the block choice.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch

from . import attention as attn_ops


@dataclass
class NSAParams:
    block_size: int = 64
    compress_type: str = "weightedpool"  # weightedpool | linear | avgpool
    kernel_size: int = 32
    kernel_stride: int = 16
    topk: int = 16
    init_blocks: int = 1
    local_blocks: int = 2
    window_size: int = 512


def compress_weight(kind: str, n_kv: int, head_dim: int, kernel: int) -> Optional[torch.Tensor]:
    """Initial value of the pooling parameter of a branch (``None`` for plain averaging)."""
    if kind == "avgpool":
        return None
    if kind == "weightedpool":
        return torch.full((n_kv, kernel), 1.0 / kernel)
    if kind == "linear":
        w = torch.zeros(n_kv, kernel, head_dim, head_dim)
        w += torch.eye(head_dim) / kernel  # starts as the window average
        return w.view(n_kv, kernel * head_dim, head_dim)
    raise ValueError(f"unknown compress_type {kind}")


def _doc_lens(cu) -> List[int]:
    c = cu.tolist() if torch.is_tensor(cu) else list(cu)
    return [int(b - a) for a, b in zip(c[:-1], c[1:])]


def compress(x: torch.Tensor, w: Optional[torch.Tensor], cu, kernel: int, stride: int,
             pe: Optional[torch.Tensor] = None, kind: str = "weightedpool") -> Tuple[torch.Tensor, List[int]]:
    """``x [T, Hkv, D]`` -> one row per complete window of every document, and the rows per document."""
    lens = _doc_lens(cu)
    starts, counts, at = [], [], 0
    for L in lens:
        n = (L - kernel) // stride + 1 if L >= kernel else 0
        starts += [at + j * stride for j in range(n)]
        counts.append(n)
        at += L
    T, H, D = x.shape
    if not starts:
        return x.new_zeros((0, H, D)), counts
    idx = torch.tensor(starts, device=x.device).unsqueeze(1) + torch.arange(kernel, device=x.device)
    win = x.index_select(0, idx.reshape(-1)).view(len(starts), kernel, H, D)
    if pe is not None:
        win = win + pe.transpose(0, 1).to(win.dtype)  # [kernel, H, D]
    if kind == "avgpool" or w is None:
        out = win.mean(1)
    elif kind == "weightedpool":
        out = torch.einsum("jkhd,hk->jhd", win, w.to(win.dtype))
    else:
        out = torch.einsum("jkhd,hkde->jhe", win, w.to(win.dtype).view(H, kernel, D, D))
    return out, counts


def _overlap_weights(block: int, kernel: int, stride: int) -> List[Tuple[int, int]]:
    """``(offset, count)``: window ``b * block/stride + offset`` shares ``count`` stride-sized pieces with
    selection block ``b``."""
    per_block, per_kernel = block // stride, kernel // stride
    counts = {}
    for piece in range(per_block):
        for part in range(per_kernel):
            counts[piece - part] = counts.get(piece - part, 0) + 1
    return sorted(counts.items())


def compressed_attention(q, k_cmp, v_cmp, cu, counts, p: NSAParams, scale: float):
    """Compressed branch.  Returns the output ``[T, Hq, D]`` and the chosen blocks ``[T, Hkv, topk]``
    (document-local block numbers, -1 where a query has fewer visible blocks)."""
    T, Hq, D = q.shape
    Hkv = k_cmp.shape[1] if k_cmp.numel() else v_cmp.shape[1]
    G = Hq // Hkv
    out = q.new_zeros((T, Hq, D))
    topk_idx = torch.full((T, Hkv, p.topk), -1, dtype=torch.long, device=q.device)
    weights = _overlap_weights(p.block_size, p.kernel_size, p.kernel_stride)
    per_block = p.block_size // p.kernel_stride
    at = ac = 0
    for L, n in zip(_doc_lens(cu), counts):
        qs = q[at:at + L].float()
        pos = torch.arange(L, device=q.device)
        nb = (L + p.block_size - 1) // p.block_size
        score = q.new_zeros((Hkv, L, nb), dtype=torch.float32)
        if n:
            kc = k_cmp[ac:ac + n].float().repeat_interleave(G, 1)
            vc = v_cmp[ac:ac + n].float().repeat_interleave(G, 1)
            ends = torch.arange(n, device=q.device) * p.kernel_stride + p.kernel_size - 1
            vis = pos[:, None] >= ends[None, :]  # [L, n]
            s = torch.einsum("qhd,khd->hqk", qs, kc) * scale
            s = s.masked_fill(~vis, float("-inf"))
            prob = torch.softmax(s, -1)
            prob = torch.nan_to_num(prob, nan=0.0)  # queries that see no finished window
            out[at:at + L] = torch.einsum("hqk,khd->qhd", prob, vc).to(out.dtype)
            pg = prob.detach().view(Hkv, G, L, n).sum(1)
            for off, cnt in weights:
                j = torch.arange(nb, device=q.device) * per_block + off
                ok = (j >= 0) & (j < n)
                if ok.any():
                    score[:, :, ok] += cnt * pg[:, :, j[ok]]
        blk = pos // p.block_size  # [L]
        b = torch.arange(nb, device=q.device)
        forced = (b[None, :] < p.init_blocks) | ((b[None, :] <= blk[:, None]) & (b[None, :] > blk[:, None] - p.local_blocks))
        score = score.masked_fill(forced.unsqueeze(0), float("inf"))
        score = score.masked_fill((b[None, :] > blk[:, None]).unsqueeze(0), float("-inf"))
        kk = min(p.topk, nb)
        val, idx = torch.topk(score, kk, dim=-1)
        idx = idx.masked_fill(val == float("-inf"), -1)
        topk_idx[at:at + L, :, :kk] = idx.permute(1, 0, 2)
        at += L
        ac += n
    return out, topk_idx


def _selected_dense(q, kf, vf, idx, block, s0, s1, G, scale):
    """Queries ``s0:s1`` of one document against all its keys under the block mask (short documents)."""
    L, Hkv = kf.shape[0], kf.shape[1]
    nb = (L + block - 1) // block
    dev = q.device
    kblk = torch.arange(L, device=dev) // block
    sel = torch.zeros((s1 - s0, Hkv, nb + 1), dtype=torch.bool, device=dev)
    sel.scatter_(2, torch.where(idx >= 0, idx, torch.full_like(idx, nb)), True)
    tok = sel[:, :, :nb].index_select(2, kblk)  # [c, Hkv, L]
    tok &= (torch.arange(L, device=dev)[None, :] <= torch.arange(s0, s1, device=dev)[:, None]).unsqueeze(1)
    tok = tok.permute(1, 0, 2).repeat_interleave(G, 0)  # [Hq, c, L]
    s = torch.einsum("qhd,khd->hqk", q, kf.repeat_interleave(G, 1)) * scale
    prob = torch.softmax(s.masked_fill(~tok, float("-inf")), -1)
    return torch.einsum("hqk,khd->qhd", prob, vf.repeat_interleave(G, 1))


def _selected_gathered(q, kf, vf, idx, block, s0, s1, G, scale):
    """The same through a gather of the chosen blocks: work grows with ``topk * block``, not with the document."""
    L, Hkv, D = kf.shape
    dev = q.device
    c, topk = s1 - s0, idx.shape[-1]
    keys = idx.clamp(min=0).unsqueeze(-1) * block + torch.arange(block, device=dev)  # [c, Hkv, topk, block]
    ok = (idx >= 0).unsqueeze(-1) & (keys <= torch.arange(s0, s1, device=dev)[:, None, None, None])
    keys = keys.clamp(max=L - 1).view(c, Hkv, topk * block)
    ok = ok.view(c, Hkv, topk * block)
    heads = torch.arange(Hkv, device=dev)[None, :, None]
    kg, vg = kf.transpose(0, 1)[heads, keys], vf.transpose(0, 1)[heads, keys]  # [c, Hkv, topk*block, D]
    qg = q.view(c, Hkv, G, D)
    s = torch.einsum("chgd,chkd->chgk", qg, kg) * scale
    prob = torch.softmax(s.masked_fill(~ok.unsqueeze(2), float("-inf")), -1)
    return torch.einsum("chgk,chkd->chgd", prob, vg).reshape(c, Hkv * G, D)


def topk_sparse_attention(q, k, v, topk_idx, block: int, cu, scale: float, q_chunk: int = 2048, gather: Optional[bool] = None):
    """Selected branch: every query attends causally to the tokens of its chosen blocks.  Documents longer than
    twice the selected span gather their blocks (``gather`` forces a path)."""
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    G = Hq // Hkv
    span = topk_idx.shape[-1] * block
    outs = []
    at = 0
    for L in _doc_lens(cu):
        kf, vf = k[at:at + L].float(), v[at:at + L].float()
        use_gather = gather if gather is not None else L > 2 * span
        step = max(1, min(q_chunk, (1 << 27) // max(1, Hkv * span * D))) if use_gather else q_chunk
        for s0 in range(0, L, step):
            s1 = min(L, s0 + step)
            fn = _selected_gathered if use_gather else _selected_dense
            outs.append(fn(q[at + s0:at + s1].float(), kf, vf, topk_idx[at + s0:at + s1], block, s0, s1, G, scale).to(q.dtype))
        at += L
    return torch.cat(outs) if outs else q.new_zeros((0, Hq, D))


def nsa_attention(q, k, v, k_cmp, v_cmp, counts, gates, cu, p: NSAParams, scale: Optional[float] = None):
    """``q [T,Hq,D]``, ``k / v [T,Hkv,D]`` (rotary applied), compressed keys / values with their rows per
    document, ``gates [T,Hq,3]`` after the sigmoid in the order (compressed, sliding, selected)."""
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    o_cmp, topk_idx = compressed_attention(q, k_cmp, v_cmp, cu, counts, p, scale)
    o_sel = topk_sparse_attention(q, k, v, topk_idx, p.block_size, cu, scale)
    cu_t = cu if torch.is_tensor(cu) else torch.tensor(cu, dtype=torch.int32, device=q.device)
    o_win = attn_ops.varlen_attn(q, k, v, cu_t, cu_t, causal=True, softmax_scale=scale, window_size=(p.window_size, -1))
    g = gates.to(q.dtype)
    return o_cmp * g[..., 0:1] + o_win * g[..., 1:2] + o_sel * g[..., 2:3]
