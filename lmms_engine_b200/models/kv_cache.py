"""Key / value cache for generation on packed streams.

Rollouts of the policy-gradient trainers (src/lmms_engine/train in the reference delegates generation to
``transformers``' ``generate`` with its ``DynamicCache``) run here on the packed varlen path: every sequence owns a slab of
``capacity`` rows in one buffer per layer; a forward pass writes the rotated keys and the values of its new tokens behind
the rows already held and attends to the gathered rows of every sequence (``cu_seqlens`` of the keys differ from those
of the queries; the attention kernel aligns its causal mask bottom-right, so new token j of a sequence sees the cached
rows and the new rows up to itself).  The gather costs one pass over the cached rows per layer and step - bandwidth
that is small against reading the layer's weights - and keeps the kernel's packed layout, so no second attention
kernel exists for decoding.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch


class PackedKVCache:
    def __init__(self, n_layers: int, capacities: Sequence[int], device=None):
        self.capacities = [int(c) for c in capacities]
        self.base = [0]
        for c in self.capacities:
            self.base.append(self.base[-1] + c)
        self.lens = [0] * len(self.capacities)
        self.k: List[Optional[torch.Tensor]] = [None] * n_layers
        self.v: List[Optional[torch.Tensor]] = [None] * n_layers
        self.device = device
        self._write = self._read = self._cu_k = None
        self._max_k = 0
        # layers that carry a recurrent state instead of keys / values (linear attention) keep it here:
        # ``state[layer][sequence]`` is whatever that layer stores (convolution tail, state matrix)
        self.state: dict = {}
        self.new_lens: List[int] = []
        self.had: List[int] = []

    def advance(self, new_lens: Sequence[int]) -> torch.Tensor:
        """Declare the next forward pass: ``new_lens[i]`` new tokens for sequence ``i`` (0 = none).  Returns the rotary
        positions of the new tokens, packed in sequence order; the pass itself is ``model(..., kv_cache=self)``."""
        new_lens = [int(n) for n in new_lens]
        if len(new_lens) != len(self.lens):
            raise ValueError(f"{len(new_lens)} lengths for a cache of {len(self.lens)} sequences")
        write, read, pos, cu = [], [], [], [0]
        self.new_lens, self.had = new_lens, list(self.lens)
        for i, n in enumerate(new_lens):
            have = self.lens[i]
            if have + n > self.capacities[i]:
                raise ValueError(f"sequence {i}: {have} cached + {n} new tokens exceed its capacity of {self.capacities[i]}")
            if n == 0:
                continue  # a sequence without new tokens has no query rows, hence no key document either
            write.append(torch.arange(self.base[i] + have, self.base[i] + have + n))
            read.append(torch.arange(self.base[i], self.base[i] + have + n))
            pos.append(torch.arange(have, have + n))
            cu.append(cu[-1] + have + n)
            self.lens[i] = have + n
        if not write:
            raise ValueError("a forward pass needs at least one new token")
        dev = self.device
        self._write, self._read = torch.cat(write).to(dev), torch.cat(read).to(dev)
        self._cu_k = torch.tensor(cu, dtype=torch.int32, device=dev)
        self._max_k = max(b - a for a, b in zip(cu[:-1], cu[1:]))
        return torch.cat(pos).to(dev)

    def extend(self, layer: int, k: torch.Tensor, v: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, int]:
        """Store this pass' keys / values of ``layer``; returns ``(keys, values, cu_seqlens_k, max_seqlen_k)`` of everything
        the new tokens attend to."""
        if self._write is None or k.shape[0] != self._write.numel():
            raise ValueError("call advance() with this pass' token counts before the forward pass")
        if self.k[layer] is None:
            self.k[layer] = k.new_zeros((self.base[-1],) + tuple(k.shape[1:]))
            self.v[layer] = v.new_zeros((self.base[-1],) + tuple(v.shape[1:]))
        self.k[layer].index_copy_(0, self._write, k.detach())
        self.v[layer].index_copy_(0, self._write, v.detach())
        return self.k[layer].index_select(0, self._read), self.v[layer].index_select(0, self._read), self._cu_k, self._max_k
