"""Pydantic base for every config object (reference: src/lmms_engine/protocol/args.py:6-13)."""
from typing import Any, Dict

from pydantic import BaseModel


class Args(BaseModel):
    extra_kwargs: Dict[str, Any] = {}

    def to_dict(self) -> Dict[str, Any]:
        return self.model_dump()

    def to_json(self) -> str:
        return self.model_dump_json()
