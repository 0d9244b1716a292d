"""Tokenizer access for processors: a Hugging Face tokenizer when ``processor_name`` is a
local path / cached model, else the built-in byte-level ChatML tokenizer (256 byte ids plus
the ChatML and vision special tokens), which keeps every data path usable offline."""
from __future__ import annotations

import json
import os
from typing import Dict, Iterable, List, Optional

SPECIAL_TOKENS = ["<|endoftext|>", "<|im_start|>", "<|im_end|>", "<|vision_start|>", "<|vision_end|>", "<|image_pad|>",
                  "<|video_pad|>", "<|AUDIO|>", "<|audio_bos|>", "<|audio_eos|>", "<|vision_pad|>"]


class ByteChatTokenizer:
    """Bytes 0..255 are ids 0..255; special tokens follow.  Lossless, no vocabulary file."""

    padding_side = "right"

    def __init__(self, extra_special: Iterable[str] = ()):
        self.special: List[str] = list(SPECIAL_TOKENS) + [t for t in extra_special if t not in SPECIAL_TOKENS]
        self._tok2id: Dict[str, int] = {t: 256 + i for i, t in enumerate(self.special)}
        self._id2tok = {v: k for k, v in self._tok2id.items()}
        self.pad_token, self.eos_token = "<|endoftext|>", "<|im_end|>"
        self.pad_token_id, self.eos_token_id = self._tok2id[self.pad_token], self._tok2id[self.eos_token]

    def __len__(self):
        return 256 + len(self.special)

    @property
    def vocab_size(self):
        return len(self)

    def convert_tokens_to_ids(self, tok):
        if isinstance(tok, (list, tuple)):
            return [self.convert_tokens_to_ids(t) for t in tok]
        return self._tok2id.get(tok, None)

    def encode(self, text: str, add_special_tokens: bool = False) -> List[int]:
        out: List[int] = []
        i = 0
        while i < len(text):
            if text[i] == "<":
                hit = next((t for t in self.special if text.startswith(t, i)), None)
                if hit is not None:
                    out.append(self._tok2id[hit])
                    i += len(hit)
                    continue
            j = i + 1
            while j < len(text) and text[j] != "<":
                j += 1
            out.extend(text[i:j].encode("utf-8"))
            i = j
        return out

    def __call__(self, text, **kw):
        if isinstance(text, str):
            return {"input_ids": self.encode(text)}
        return {"input_ids": [self.encode(t) for t in text]}

    def decode(self, ids, skip_special_tokens: bool = False) -> str:
        parts, buf = [], bytearray()
        for i in (ids.tolist() if hasattr(ids, "tolist") else ids):
            if i < 256:
                buf.append(i)
            else:
                if buf:
                    parts.append(buf.decode("utf-8", errors="replace"))
                    buf = bytearray()
                if not skip_special_tokens:
                    parts.append(self._id2tok.get(i, ""))
        if buf:
            parts.append(buf.decode("utf-8", errors="replace"))
        return "".join(parts)

    def batch_decode(self, batch, **kw):
        return [self.decode(x, **kw) for x in batch]

    def save_pretrained(self, path: str):
        os.makedirs(path, exist_ok=True)
        with open(os.path.join(path, "byte_chat_tokenizer.json"), "w") as f:
            json.dump({"type": "byte_chat", "special_tokens": self.special}, f)


REALTIME_TOKENS = ["<|audio_start|>", "<|audio_end|>", "<|audio_pad|>", "<|rt_start|>", "<|rt_pad|>", "<|rt_speak|>", "<|rt_end|>"]


def load_tokenizer(name: Optional[str]):
    if name == "byte_realtime":
        return ByteChatTokenizer(REALTIME_TOKENS)
    if not name or name in ("byte", "none", "byte_chat"):
        return ByteChatTokenizer()
    marker = os.path.join(name, "byte_chat_tokenizer.json") if os.path.isdir(name) else None
    if marker and os.path.exists(marker):
        with open(marker) as f:
            return ByteChatTokenizer(json.load(f).get("special_tokens", ()))
    from transformers import AutoTokenizer

    return AutoTokenizer.from_pretrained(name)
