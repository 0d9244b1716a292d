"""Map-style multimodal SFT dataset with offline packing
(reference: src/lmms_engine/datasets/naive/multimodal_dataset.py:31-411): shuffle, token-length
estimate per record, overlong filtering, ``first_fit`` / ``window_N`` packing into index
groups, ``modality_length`` for length-grouped sampling."""
from __future__ import annotations

import random
from typing import Dict, List

import torch
from torch.utils.data import Dataset

from ...mapping_func import register_dataset
from ...utils.logging_utils import logger
from ..base import DatasetCore
from ..packing import build_offline_groups


class MultiModalDataset(DatasetCore, Dataset):
    def build(self):
        super().build()
        cfg = self.config
        order = list(range(len(self.data_list)))
        if cfg.shuffle:
            random.Random(cfg.data_seed or 0).shuffle(order)
        self.data_list = [self.data_list[i] for i in order]
        self.data_folder = [self.data_folder[i] for i in order]
        self.lengths = [self.estimate_tokens(r) for r in self.data_list]
        limit = cfg.packing_length if cfg.packing else cfg.max_length
        if cfg.filter_overlong and limit:
            keep = [i for i, n in enumerate(self.lengths) if n <= limit]
            if len(keep) != len(self.lengths):
                logger.info(f"filtered {len(self.lengths) - len(keep)} overlong records (> {limit} estimated tokens)")
            self.data_list = [self.data_list[i] for i in keep]
            self.data_folder = [self.data_folder[i] for i in keep]
            self.lengths = [self.lengths[i] for i in keep]
        if cfg.packing:
            self.groups = build_offline_groups(cfg.packing_strategy or "first_fit", self.lengths, cfg.packing_length)
        else:
            self.groups = [[i] for i in range(len(self.data_list))]
        return self

    @property
    def modality_length(self) -> List[int]:
        """Signed group lengths: positive when the group holds media, negative for text only."""
        out = []
        for g in self.groups:
            n = sum(self.lengths[i] for i in g)
            has_mm = any(any(c.get("type") != "text" for m in self.messages_of(self.data_list[i])
                             for c in (m["content"] if isinstance(m["content"], list) else [])) for i in g)
            out.append(n if has_mm else -n)
        return out

    def __len__(self):
        return len(self.groups)

    def __getitem__(self, idx) -> List[Dict[str, torch.Tensor]]:
        return [self.process_record(self.data_list[i], self.data_folder[i]) for i in self.groups[idx]]


# ``vision``, ``vision_audio`` and ``text`` differ in the reference only by which media their records hold, which the
# generic record handling discovers by itself; datasets with behaviour of their own live in ``datasets/families.py``
for _name in ("vision", "vision_audio", "text"):
    register_dataset(_name)(type(f"{_name.title().replace('_', '')}Dataset", (MultiModalDataset,), {"__doc__": f"``dataset_type: {_name}``"}))
