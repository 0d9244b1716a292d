"""Multimodal rotary position ids ``[3, T]`` (temporal, height, width) for packed streams.

Text tokens advance all three streams together.  A run of vision placeholder tokens that
stands for a ``(t, h, w)`` patch grid (``h/m x w/m`` merged tokens per temporal step) gets the
temporal index ``floor(frame * seconds_per_grid * tokens_per_second)`` (0 for images and for
Qwen3-VL, whose frames are separated by timestamp text), the row index and the column index
of each merged token, all offset by the running position; text after the run resumes at
``max(position) + 1``.  Every document of a packed stream restarts at 0.  Host-side numpy;
behaviour of ``qwen2_5_vl_rope_index`` / ``qwen3_vl_get_rope_index`` in the reference
(src/lmms_engine/models/common_ops/rope.py:8-346).
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch


def _runs(mask: np.ndarray) -> List[Tuple[int, int]]:
    if not mask.any():
        return []
    d = np.diff(np.concatenate([[0], mask.astype(np.int8), [0]]))
    return list(zip(np.nonzero(d == 1)[0].tolist(), np.nonzero(d == -1)[0].tolist()))


def mrope_positions_one(ids: np.ndarray, vision_ids: Sequence[int], grids: List[Tuple[int, int, int]],
                        seconds: Optional[List[float]], merge: int, tokens_per_second: float) -> Tuple[np.ndarray, int]:
    """Positions ``[3, n]`` of one document and the number of grids consumed."""
    n = ids.shape[0]
    pos = np.zeros((3, n), dtype=np.int64)
    is_vis = np.isin(ids, np.asarray(list(vision_ids)))
    cur = 0  # next position value
    at = 0  # cursor in the stream
    used = 0
    for lo, hi in _runs(is_vis):
        # text before the run
        if lo > at:
            pos[:, at:lo] = np.arange(lo - at)[None] + cur
            cur += lo - at
        p = lo
        while p < hi:
            if used >= len(grids):
                raise ValueError("more vision placeholder runs than grids")
            t, h, w = grids[used]
            gh, gw = h // merge, w // merge
            cnt = t * gh * gw
            if p + cnt > hi:
                raise ValueError(f"placeholder run of {hi - p} tokens does not match grid {grids[used]} ({cnt} tokens)")
            sec = seconds[used] if seconds is not None else 0.0
            ti = np.floor(np.arange(t) * sec * tokens_per_second).astype(np.int64)
            pos[0, p:p + cnt] = np.repeat(ti, gh * gw) + cur
            pos[1, p:p + cnt] = np.tile(np.repeat(np.arange(gh), gw), t) + cur
            pos[2, p:p + cnt] = np.tile(np.arange(gw), t * gh) + cur
            cur = int(pos[:, p:p + cnt].max()) + 1
            p += cnt
            used += 1
        at = hi
    if at < n:
        pos[:, at:] = np.arange(n - at)[None] + cur
    return pos, used


def build_mrope_positions(input_ids, cu_seqlens, vision_token_ids: Sequence[int], grids, seconds=None, merge: int = 2,
                          tokens_per_second: float = 0.0) -> torch.Tensor:
    """Positions for a packed stream: ``input_ids [T]``, ``cu_seqlens [n+1]``; ``grids`` lists the
    ``(t, h, w)`` of every image / video in order of appearance over the whole stream."""
    ids = input_ids.cpu().numpy() if torch.is_tensor(input_ids) else np.asarray(input_ids)
    cu = cu_seqlens.cpu().tolist() if torch.is_tensor(cu_seqlens) else list(cu_seqlens)
    grids = [(int(a), int(b), int(c)) for a, b, c in (grids.tolist() if torch.is_tensor(grids) else grids)]
    seconds = list(seconds.tolist() if torch.is_tensor(seconds) else seconds) if seconds is not None else None
    out = np.zeros((3, ids.shape[0]), dtype=np.int64)
    g = 0
    for d in range(len(cu) - 1):
        lo, hi = cu[d], cu[d + 1]
        pos, used = mrope_positions_one(ids[lo:hi], vision_token_ids, grids[g:], seconds[g:] if seconds is not None else None,
                                        merge, tokens_per_second)
        out[:, lo:hi] = pos
        g += used
    return torch.from_numpy(out)


# ---------------------------------------------------------------------------------------------
# Qwen2.5-Omni: a video whose sound track is used ("use_audio_in_video") is written as
#   <vision_bos><audio_bos> [video chunk 0][audio chunk 0][video chunk 1][audio chunk 1]... <audio_eos><vision_eos>
# where a chunk holds the tokens of ``seconds_per_chunk`` seconds (``position_id_per_seconds`` positions per
# second).  Both modalities count time from the same origin, so tokens of one moment share temporal positions.
def chunked_index(values: np.ndarray, per_chunk: int) -> List[Tuple[int, int]]:
    """Slices ``[start, end)`` of a non-decreasing sequence whose values fall into successive ranges of
    ``per_chunk``: ``[0, per_chunk)``, ``[per_chunk, 2 per_chunk)``, ...  (empty ranges yield no slice of their own:
    a slice ends where the value first reaches the next multiple)."""
    out, start, chunk = [], 0, 1
    for i, v in enumerate(values.tolist()):
        if v >= chunk * per_chunk:
            out.append((start, i))
            start = i
            chunk += 1
    out.append((start, len(values)))
    return out


def interleave_av(video_t: np.ndarray, n_audio: int, per_chunk: int) -> List[Tuple[str, int, int]]:
    """Order of the chunks of one audio-visual block: ``("video" | "audio", start, end)`` slices into the
    modality's own token sequence.  ``video_t`` holds the temporal position (relative to the block's origin) of
    every video token."""
    v_chunks = chunked_index(video_t, per_chunk)
    a_chunks = chunked_index(np.arange(n_audio), per_chunk)
    order = []
    for j in range(max(len(v_chunks), len(a_chunks))):
        if j < len(v_chunks):
            order.append(("video",) + v_chunks[j])
        if j < len(a_chunks):
            order.append(("audio",) + a_chunks[j])
    return order


def omni_positions_one(ids: np.ndarray, image_id: int, video_id: int, audio_id: int, image_grids, video_grids, video_seconds,
                       merge: int, tokens_per_second: float, seconds_per_chunk: float = 2.0) -> np.ndarray:
    """``[3, n]`` positions of one Qwen2.5-Omni document in which every video carries its sound track
    (runs that mix video and audio placeholders).  Images, sound-less videos and stand-alone audio clips are
    positioned as everywhere else (audio tokens count like text).  Follows the upstream index
    (transformers ``Qwen2_5OmniPreTrainedModelForConditionalGeneration.get_rope_index``) including two of
    its conventions: the two begin tokens of a block share one position, as do its two end tokens, and the
    position after a block continues from the block's LAST chunk, not from its largest position."""
    n = ids.shape[0]
    pos = np.zeros((3, n), dtype=np.int64)
    per_chunk = int(tokens_per_second * seconds_per_chunk)
    cur, p, ii, vi = 0, 0, 0, 0
    special = np.isin(ids, [image_id, video_id, audio_id])

    def text(lo, hi):
        nonlocal cur
        if hi > lo:
            pos[:, lo:hi] = np.arange(hi - lo)[None] + cur
            cur += hi - lo

    def vision(t, h, w, sec, origin):
        gh, gw = h // merge, w // merge
        ti = np.floor(np.arange(t) * sec * tokens_per_second).astype(np.int64)
        return np.stack([np.repeat(ti, gh * gw), np.tile(np.repeat(np.arange(gh), gw), t), np.tile(np.arange(gw), t * gh)]) + origin

    while p < n:
        nxt = np.nonzero(special[p:])[0]
        if nxt.size == 0:
            text(p, n)
            break
        q = p + int(nxt[0])
        if ids[q] == image_id:
            text(p, q)
            t, h, w = image_grids[ii]
            ii += 1
            cnt = t * (h // merge) * (w // merge)
            pos[:, q:q + cnt] = vision(t, h, w, 1.0, cur)
            cur = int(pos[:, q:q + cnt].max()) + 1
            p = q + cnt
            continue
        r = q
        while r < n and ids[r] in (video_id, audio_id):
            r += 1
        is_v = ids[q:r] == video_id
        n_v, n_a = int(is_v.sum()), int((~is_v).sum())
        if n_v == 0:  # a stand-alone audio clip
            text(p, r)
            p = r
            continue
        t, h, w = video_grids[vi]
        sec = video_seconds[vi] if video_seconds is not None else 1.0
        vi += 1
        if n_v != t * (h // merge) * (w // merge):
            raise ValueError(f"run of {n_v} video tokens does not match grid {(t, h, w)}")
        if n_a == 0:  # a video without sound
            text(p, q)
            pos[:, q:r] = vision(t, h, w, sec, cur)
            cur = int(pos[:, q:r].max()) + 1
            p = r
            continue
        # audio-visual block: [q - 2, q) are the two begin tokens, [r, r + 2) the two end tokens
        text(p, q - 2)
        pos[:, q - 2:q] = cur
        cur += 1
        vpos = vision(t, h, w, sec, cur)
        apos = np.arange(n_a)[None].repeat(3, 0) + cur
        pos[:, q:r][:, is_v] = vpos
        pos[:, q:r][:, ~is_v] = apos
        kind, lo, hi = interleave_av(vpos[0] - cur, n_a, per_chunk)[-1]
        cur = int((vpos if kind == "video" else apos)[:, lo:hi].max()) + 1
        pos[:, r:r + 2] = cur
        cur += 1
        p = r + 2
    return pos
