"""Masked-diffusion language models (``qwen3_dllm`` / ``dream_dllm`` / ``llada_dllm``): the
packed decoder with bidirectional attention; a random fraction ``t`` of each sequence is
replaced by the mask token and the loss is the cross-entropy on masked positions weighted by
``1/t``.  Returns ``loss`` (the diffusion objective) and ``nll`` (unweighted masked-token CE), as the
reference models do (src/lmms_engine/models/qwen3_dllm/modeling_qwen3_dllm.py:47-95, 539-556)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional

import torch

from ..ops import cross_entropy as ce_ops
from .decoder_lm import IGNORE_INDEX, DecoderConfig, DecoderLM, _w


@dataclass
class DLLMConfig(DecoderConfig):
    model_type: str = "qwen3_dllm"
    mask_token_id: int = 151666

    def __post_init__(self):
        super().__post_init__()
        if self.model_type == "qwen3_dllm":
            self.qk_norm = True
        self.architectures = [{"qwen3_dllm": "Qwen3DLLMForMaskedLM", "dream_dllm": "DreamDLLMForMaskedLM",
                               "llada_dllm": "LLaDADLLMForMaskedLM"}.get(self.model_type, "Qwen3DLLMForMaskedLM")]


class DiffusionLM(DecoderLM):
    supports_kv_cache = False
    config_class = DLLMConfig

    def __init__(self, cfg: DLLMConfig):
        super().__init__(cfg)
        self.causal = False
        self.shift_labels = False

    def forward(self, input_ids=None, labels=None, mlm_prob: Optional[torch.Tensor] = None, **kw) -> Dict[str, Any]:
        """``input_ids`` already carry mask tokens; ``labels`` hold the original id at masked positions
        and -100 elsewhere; ``mlm_prob`` is the per-token masking ratio ``t`` of its sequence."""
        out = super().forward(input_ids=input_ids, labels=None, **kw)
        hidden = out["hidden_states"]
        if labels is None:
            return out
        lab = labels.reshape(-1)
        per_tok = ce_ops.fused_linear_cross_entropy(hidden, _w(self.lm_head.weight), lab, "none")
        valid = (lab != IGNORE_INDEX).to(per_tok.dtype)
        n = valid.sum().clamp(min=1.0)
        nll = (per_tok * valid).sum() / n
        if mlm_prob is not None:
            t = mlm_prob.reshape(-1).to(per_tok.dtype).clamp(min=1e-3)
            loss = (per_tok * valid / t).sum() / lab.numel()
        else:
            loss = nll
        out.update(loss=loss, nll=nll.detach(), hidden_states=None)
        return out
