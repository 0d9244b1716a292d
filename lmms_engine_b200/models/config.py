"""Model section of the YAML (reference: src/lmms_engine/models/config.py:6-18)."""
from typing import Any, Dict, Literal, Optional

from ..protocol import Args


class ModelConfig(Args):
    load_from_pretrained_path: Optional[str] = None
    load_from_config: Optional[Dict[str, Any]] = None
    attn_implementation: Optional[Literal["flash_attention_2", "sdpa", "eager", "b200"]] = "sdpa"
    model_general_type: Optional[Literal["causal_lm", "masked_lm", "image_text_to_text", "general"]] = None
    overwrite_config: Optional[Dict[str, Any]] = None
    monkey_patch_kwargs: Optional[Dict[str, Any]] = None
