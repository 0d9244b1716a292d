"""Samplers of the map-style training path.

``LengthGroupedSampler`` keeps the samples of one optimizer step similar in length, so that padded
batches waste little and data-parallel ranks finish their micro-batches together.  It plays the role
of the length-grouped samplers that the reference's HF trainer takes from ``transformers``
(src/lmms_engine/train/hf/trainer.py:145-188: ``LengthGroupedSampler`` /
``DistributedLengthGroupedSampler`` over ``dataset.modality_length``) with one sampler for both
cases: it is aware of the data-parallel layout (ranks of one sequence-parallel group share a
data-parallel rank and therefore draw the same samples).

Algorithm: a seeded permutation is cut into windows of ``window_batches`` global batches; inside a
window, multimodal samples (positive ``modality_length``) and text-only samples (negative) are
sorted by length separately and chopped into global batches of ``batch_size * num_replicas``; the
batches of a window are then shuffled.  A rank takes a strided slice of every global batch, so the
ranks of a step hold neighbours in the length order.
"""
from __future__ import annotations

from typing import Iterator, List, Optional, Sequence

import torch
from torch.utils.data import Sampler


class LengthGroupedSampler(Sampler[int]):
    def __init__(self, lengths: Sequence[int], batch_size: int, num_replicas: int = 1, rank: int = 0, seed: int = 0,
                 window_batches: int = 50, drop_last: bool = False):
        if not 0 <= rank < num_replicas:
            raise ValueError(f"rank {rank} outside [0, {num_replicas})")
        self.lengths = [int(x) for x in lengths]
        self.batch_size = max(int(batch_size), 1)
        self.num_replicas, self.rank = int(num_replicas), int(rank)
        self.seed, self.epoch = int(seed), 0
        self.window_batches = max(int(window_batches), 1)
        self.drop_last = drop_last
        g = self.batch_size * self.num_replicas
        n = len(self.lengths)
        self.num_global_batches = n // g if drop_last else -(-n // g)

    def set_epoch(self, epoch: int) -> None:
        self.epoch = int(epoch)

    def __len__(self) -> int:
        return self.num_global_batches * self.batch_size

    def global_batches(self) -> List[List[int]]:
        """Global batches of one epoch (identical on every rank)."""
        gen = torch.Generator().manual_seed(self.seed + self.epoch)
        n = len(self.lengths)
        g = self.batch_size * self.num_replicas
        perm = torch.randperm(n, generator=gen).tolist()
        if not self.drop_last and n % g:
            perm += perm[: g - n % g]  # wrap around so that every rank gets full batches
        elif self.drop_last:
            perm = perm[: n - n % g]
        window = g * self.window_batches
        out: List[List[int]] = []
        for w0 in range(0, len(perm), window):
            chunk = perm[w0 : w0 + window]
            mm = sorted((i for i in chunk if self.lengths[i] >= 0), key=lambda i: -self.lengths[i])
            tx = sorted((i for i in chunk if self.lengths[i] < 0), key=lambda i: self.lengths[i])
            batches = [mm[i : i + g] for i in range(0, len(mm) - len(mm) % g, g)]
            batches += [tx[i : i + g] for i in range(0, len(tx) - len(tx) % g, g)]
            rest = mm[len(mm) - len(mm) % g :] + tx[len(tx) - len(tx) % g :]  # a mixed batch at most once per window
            batches += [rest[i : i + g] for i in range(0, len(rest), g)]
            order = torch.randperm(len(batches), generator=gen).tolist()
            out += [batches[j] for j in order]
        return [b for b in out if len(b) == g]

    def __iter__(self) -> Iterator[int]:
        for batch in self.global_batches():
            # strided slice: rank r takes elements r, r + R, ... of the length-sorted batch
            yield from batch[self.rank :: self.num_replicas]


def dataset_lengths(dataset) -> Optional[List[int]]:
    """``modality_length`` (sign marks text-only samples) or ``lengths`` of a dataset, if it has them."""
    for attr in ("modality_length", "lengths"):
        v = getattr(dataset, attr, None)
        if v is not None:
            v = v() if callable(v) else v
            return list(v)
    return None
