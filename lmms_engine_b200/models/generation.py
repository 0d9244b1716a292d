"""Generation on the packed key / value cache for the decoder and vision-language families, and the streaming
session of the realtime model.

The reference generates through ``transformers.GenerationMixin`` with its ``DynamicCache`` (patched models) and keeps
hand-written caches in its in-repo models (src/lmms_engine/models/aero_realtime/modeling_aero_realtime.py:700-1385: audio
encoder convolution cache, per-chunk decoding).  Here one mechanism serves all of them: the prompt - with its images,
videos and audio - runs once through the ordinary forward pass with ``kv_cache=PackedKVCache`` (models/kv_cache.py), which
records every layer's rotated keys and values; each following step feeds one token (the realtime session: one audio
slot) at the next rotary position.

Rotary positions of multimodal prompts are not the token index (an image occupies one temporal position), so the
position of the first generated token is read from the positions the model itself built for the prompt: largest
position + 1, on all three axes.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional

import torch
import torch.nn.functional as F

from .kv_cache import PackedKVCache


def _decoder(model):
    """The causal LM that owns the layers: the model itself, or the ``language_model`` of a multimodal wrapper."""
    return getattr(model, "language_model", model)


def _prompt_positions(model, run) -> torch.Tensor:
    """Run ``run()`` (a forward pass of ``model``) and return the ``position_ids`` its decoder received."""
    seen: Dict[str, Any] = {}
    lm = _decoder(model)

    def grab(_module, args, kwargs):
        if kwargs.get("position_ids") is not None:
            seen["pos"] = kwargs["position_ids"]

    handle = lm.register_forward_pre_hook(grab, with_kwargs=True)
    try:
        seen["out"] = run()
    finally:
        handle.remove()
    return seen.get("pos"), seen["out"]


def _next_token(model, hidden_last: torch.Tensor, temperature: float, generator) -> torch.Tensor:
    head = _decoder(model).lm_head.weight
    if hasattr(head, "full_tensor"):  # held in shards by a wrapper outside the forward pass
        head = head.full_tensor()
    logits = F.linear(hidden_last, head).float()
    if temperature and temperature > 0:
        return torch.multinomial(torch.softmax(logits / temperature, -1), 1, generator=generator).flatten()
    return logits.argmax(-1)


class GenerationState:
    """Cache, next rotary position and last hidden row of ONE sequence."""

    def __init__(self, model, capacity: int, device):
        lm = _decoder(model)
        if not getattr(lm, "supports_kv_cache", False):
            raise NotImplementedError(f"{type(lm).__name__} has no key / value cache path")
        self.model = model
        self.cache = PackedKVCache(len(lm.model.layers), [capacity], device=device)
        self.next_pos = 0
        self.mrope = False
        self.device = device

    def prefill(self, input_ids: torch.Tensor, **inputs) -> torch.Tensor:
        """Run the prompt (``input_ids [T]`` plus the model's multimodal inputs); returns the hidden state of its last
        token."""
        ids = input_ids.reshape(-1)
        n = ids.numel()
        plain = self.cache.advance([n])
        cu = torch.tensor([0, n], dtype=torch.int32, device=ids.device)
        multimodal = _decoder(self.model) is not self.model
        kw = dict(inputs) if multimodal else dict(inputs, position_ids=plain)
        pos, out = _prompt_positions(self.model, lambda: self.model(input_ids=ids, cu_seqlens=cu, kv_cache=self.cache, **kw))
        pos = plain if pos is None else pos
        self.mrope = pos.dim() == 2
        self.next_pos = int(pos.max()) + 1
        return out["hidden_states"][-1:]

    def step(self, token: torch.Tensor, **inputs) -> torch.Tensor:
        """Feed one token (``[1]``; with ``inputs`` e.g. one audio slot's features); returns its hidden state."""
        self.cache.advance([1])
        p = torch.full((3, 1) if self.mrope else (1,), self.next_pos, dtype=torch.long, device=token.device)
        self.next_pos += 1
        cu = torch.tensor([0, 1], dtype=torch.int32, device=token.device)
        return self.model(input_ids=token.reshape(1), cu_seqlens=cu, position_ids=p, kv_cache=self.cache, **inputs)["hidden_states"]


@torch.no_grad()
def generate(model, input_ids: torch.Tensor, max_new_tokens: int, eos_token_id: Optional[int] = None, temperature: float = 0.0,
             generator=None, **inputs) -> torch.Tensor:
    """Continue ONE sequence: ``input_ids [T]`` (or ``[1, T]``) with the model's other inputs (``pixel_values``,
    ``image_grid_thw``, ``input_features``, ``text_stream_ids`` ...).  Greedy for ``temperature`` 0, ancestral sampling
    otherwise.  Returns the new tokens."""
    ids = input_ids.reshape(-1)
    state = GenerationState(model, ids.numel() + max_new_tokens, ids.device)
    for name in ("text_stream_ids",):
        if inputs.get(name) is not None:
            inputs[name] = inputs[name].reshape(-1)
    hidden = state.prefill(ids, **inputs)
    new: List[torch.Tensor] = []
    for i in range(max_new_tokens):
        tok = _next_token(model, hidden, temperature, generator)
        new.append(tok)
        if (eos_token_id is not None and int(tok) == eos_token_id) or i == max_new_tokens - 1:
            break
        hidden = state.step(tok)
    return torch.cat(new) if new else ids.new_zeros((0,))


class RealtimeSession:
    """Streaming inference of the realtime model: after the prompt, every call of ``listen`` brings the mel features of
    one audio slot (``[n_mels, 2 * downsample_factor]``) and returns the token the model emits for that slot -
    ``<|rt_pad|>`` while it stays silent, speech tokens otherwise.  The emitted token is what the text stream carries at
    the NEXT slot, as in training, where the stream at a slot holds the token spoken there and the label of a slot is the
    stream's next entry.

    ``continuous_audio = False``: every slot is encoded by itself (a model trained on the ``chunk_audio`` layout of the
    processor).  ``True``: the slots are pieces of one clip - the audio encoder continues from its convolution tails and
    its keys / values of the earlier slots, so slot t is encoded exactly as inside the whole clip (a model trained on whole
    clips; the reference's padding cache plus encoder cache)."""

    def __init__(self, model, rt_pad_id: int, audio_start_id: Optional[int] = None, max_slots: int = 4096,
                 continuous_audio: bool = False):
        self.model, self.rt_pad = model, int(rt_pad_id)
        self.continuous_audio = continuous_audio
        self.audio_cache = None
        self.audio_start = audio_start_id
        self.max_slots = max_slots
        self.state: Optional[GenerationState] = None
        self.last: Optional[torch.Tensor] = None
        self.hidden: Optional[torch.Tensor] = None

    @torch.no_grad()
    def start(self, prompt_ids: torch.Tensor, **inputs) -> None:
        """``prompt_ids``: everything up to and including ``<|audio_start|>`` of the stream that is about to begin."""
        ids = prompt_ids.reshape(-1)
        self.state = GenerationState(self.model, ids.numel() + self.max_slots, ids.device)
        self.hidden = self.state.prefill(ids, **inputs)
        self.audio_cache = self.model.audio_tower.new_stream() if self.continuous_audio else None
        self.last = _next_token(self.model, self.hidden, 0.0, None)  # what the stream carries at the first slot

    @torch.no_grad()
    def listen(self, slot_features: torch.Tensor, temperature: float = 0.0, generator=None) -> int:
        cfg = self.model.config
        dev = self.last.device
        feats = slot_features.reshape(1, slot_features.shape[-2], slot_features.shape[-1]).to(dev)
        mask = torch.ones((1, feats.shape[-1] // 2), dtype=torch.long, device=dev)
        slot = torch.tensor([cfg.audio_token_id], device=dev)
        extra = {"audio_stream_cache": self.audio_cache} if self.audio_cache is not None else {}
        self.hidden = self.state.step(slot, text_stream_ids=self.last, input_features=feats, audio_attention_mask=mask, **extra)
        self.last = _next_token(self.model, self.hidden, temperature, generator)
        return int(self.last)
