"""Streaming multimodal dataset (reference:
src/lmms_engine/datasets/iterable/multimodal_iterable_dataset.py:34-281): deterministic seeded
shuffle, contiguous shard per data-parallel rank then per dataloader worker, ONLINE packing
through a strategy object, oversize samples bypass the packer, records that fail to process are
skipped with a log line, ``state_dict`` / ``load_state_dict`` (``cur_idx``) for resumable loaders."""
from __future__ import annotations

import random
from typing import Any, Dict, Iterator, List

import torch
from torch.utils.data import IterableDataset, get_worker_info

from ...mapping_func import register_dataset
from ...utils.logging_utils import logger
from ..base import DatasetCore
from ..packing import build_online_packer


class MultiModalIterableDataset(DatasetCore, IterableDataset):
    def __init__(self, config):
        super().__init__(config)
        self.cur_idx = 0
        # set by load_state_dict and cleared by the next __iter__: that pass continues from the
        # restored cursor, every other pass starts at the beginning of the shard
        self._resuming = False
        self.dp_rank, self.dp_size = 0, 1

    def build(self):
        super().build()
        cfg = self.config
        order = list(range(len(self.data_list)))
        if cfg.shuffle:
            random.Random(cfg.data_seed or 0).shuffle(order)
        self.order = order
        try:
            from ...parallel import process_group_manager as pgm

            if pgm.process_group_manager is not None:
                self.dp_rank, self.dp_size = pgm.process_group_manager.dp_rank, pgm.process_group_manager.dp_size
        except Exception:
            pass
        return self

    def state_dict(self) -> Dict[str, Any]:
        return {"cur_idx": self.cur_idx}

    def load_state_dict(self, sd: Dict[str, Any]) -> None:
        self.cur_idx = int(sd.get("cur_idx", 0))
        self._resuming = True

    def _my_indices(self) -> List[int]:
        """Contiguous shard of the shuffled order for this data-parallel rank (the first
        ``n % dp_size`` ranks hold one record more, so no record is dropped), then a contiguous
        slice of ``ceil(len / workers)`` records per dataloader worker."""
        n = len(self.order)
        base, extra = divmod(n, self.dp_size)
        start = self.dp_rank * base + min(self.dp_rank, extra)
        mine = self.order[start:start + base + (1 if self.dp_rank < extra else 0)]
        info = get_worker_info()
        if info is not None and info.num_workers > 1:
            per_w = -(-len(mine) // info.num_workers)
            mine = mine[info.id * per_w:min((info.id + 1) * per_w, len(mine))]
        return mine

    def __iter__(self) -> Iterator[List[Dict[str, torch.Tensor]]]:
        cfg = self.config
        mine = self._my_indices()
        packer = None
        if cfg.packing:
            kw = dict((cfg.extra_kwargs or {}).get("packing_kwargs", {}) or {})
            packer = build_online_packer(cfg.packing_strategy or "first_fit", cfg.packing_length, **kw)
        if not self._resuming:
            self.cur_idx = 0
        self._resuming = False
        pos = self.cur_idx
        while pos < len(mine):
            i = mine[pos]
            pos += 1
            try:
                sample = self.process_record(self.data_list[i], self.data_folder[i])
            except Exception as e:
                logger.warning(f"skipping record {i}: {type(e).__name__}: {e}")
                continue
            n = int(sample["input_ids"].numel())
            if packer is None:
                self.cur_idx = pos
                yield [sample]
                continue
            if n > cfg.packing_length:
                if cfg.filter_overlong:
                    continue
                # oversize samples bypass the packer; what it holds goes out first, so the order of
                # the stream is kept
                for pack in packer.flush():
                    self.cur_idx = pos - 1
                    yield pack
                self.cur_idx = pos
                yield [sample]
                continue
            for pack in packer.add(sample, n):
                self.cur_idx = pos - 1 if (cfg.packing_strategy or "first_fit") == "first_fit" else pos
                yield pack
        if packer is not None:
            for pack in packer.flush():
                self.cur_idx = pos
                yield pack


# generic record handling; ``qwen3_vl_iterable`` / ``qwen_omni_iterable`` are in ``datasets/families.py``,
# ``llava_ov2_iterable`` (codec-stream videos) in ``datasets/codec_video.py``
for _name in ("vision_iterable", "text_iterable"):
    register_dataset(_name)(type(f"{_name.title().replace('_', '')}Dataset", (MultiModalIterableDataset,), {"__doc__": f"``dataset_type: {_name}``"}))
