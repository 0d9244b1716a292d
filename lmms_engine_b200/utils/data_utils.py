"""Data-file loading helpers (reference: src/lmms_engine/utils/data_utils.py:69-295):
json / jsonl / csv / arrow / parquet / hf_dataset loaders, YAML multi-source lists
(``datasets: [{path, data_folder, data_type}]``) loaded in parallel and concatenated with a
``data_folder`` column, frame-count arithmetic for video sampling, retrying blob download."""
from __future__ import annotations

import io
import json
import math
import os
import time
from concurrent.futures import ThreadPoolExecutor
from typing import Any, Callable, Dict, List, Optional, Tuple

import yaml

from .logging_utils import logger

FRAME_FACTOR = 2


class DataUtilities:
    @staticmethod
    def load_json(path: str) -> List[dict]:
        with open(path) as f:
            return json.load(f)

    @staticmethod
    def load_jsonlines(path: str) -> List[dict]:
        out = []
        with open(path) as f:
            for line in f:
                line = line.strip()
                if line:
                    out.append(json.loads(line))
        return out

    @staticmethod
    def load_csv(path: str) -> List[dict]:
        import pandas as pd

        return pd.read_csv(path).to_dict("records")

    @staticmethod
    def load_table(path: str, data_type: str) -> List[dict]:
        if data_type == "parquet":
            import pyarrow.parquet as pq

            return pq.read_table(path).to_pylist()
        if data_type == "arrow":
            try:
                import datasets

                if os.path.isdir(path):
                    return datasets.load_from_disk(path).to_list()
            except ImportError:
                pass
            import pyarrow as pa

            with pa.memory_map(path) as src:
                try:
                    return pa.ipc.open_file(src).read_all().to_pylist()
                except pa.ArrowInvalid:
                    return pa.ipc.open_stream(src).read_all().to_pylist()
        raise ValueError(data_type)

    @staticmethod
    def load_one(path: str, data_type: str) -> List[dict]:
        if data_type == "json":
            return DataUtilities.load_json(path)
        if data_type == "jsonl":
            return DataUtilities.load_jsonlines(path)
        if data_type == "csv":
            return DataUtilities.load_csv(path)
        if data_type in ("arrow", "parquet"):
            return DataUtilities.load_table(path, data_type)
        if data_type == "hf_dataset":
            import datasets

            return datasets.load_dataset(path, split="train").to_list()
        raise ValueError(f"unknown data_type '{data_type}'")

    @staticmethod
    def load_yaml(path: str) -> Tuple[List[dict], List[str]]:
        with open(path) as f:
            spec = yaml.safe_load(f)
        return DataUtilities.load_inline_datasets(spec["datasets"])

    @staticmethod
    def _load_spec(spec: dict):
        return DataUtilities.load_one(spec["path"], spec.get("data_type", "json"))

    @staticmethod
    def load_inline_datasets(specs: List[dict], workers: int = 8, processes: Optional[bool] = None) -> Tuple[List[dict], List[str]]:
        """Every source is loaded in parallel; returns the concatenated records and, per record, the ``data_folder`` of
        the source it came from.  Parsing JSON holds the interpreter lock, so with several large sources the loads run
        in worker PROCESSES (like the reference's pool, src/lmms_engine/utils/data_utils.py:129-153, 235-272);
        ``processes=None`` chooses that when the sources total more than 64 MB, threads otherwise (no fork for small
        data, and tests stay cheap).  ``LMMS_B200_DATA_LOAD_PROCESSES=0|1`` overrides."""
        if not specs:
            return [], []
        env = os.environ.get("LMMS_B200_DATA_LOAD_PROCESSES")
        if env is not None:
            processes = env == "1"
        if processes is None:
            size = sum(os.path.getsize(s["path"]) for s in specs if os.path.isfile(s.get("path", "")))
            processes = len(specs) > 1 and size > 64 * 2 ** 20
        n = max(1, min(workers, len(specs)))
        if processes:
            import torch

            # forked workers are cheap and need no importable main module, but a process that already holds a CUDA
            # context must not fork: fall back to threads there
            processes = not (torch.cuda.is_available() and torch.cuda.is_initialized())
        if processes:
            import multiprocessing as mp
            from concurrent.futures import ProcessPoolExecutor

            with ProcessPoolExecutor(max_workers=n, mp_context=mp.get_context("fork")) as ex:
                parts = list(ex.map(DataUtilities._load_spec, specs))
        else:
            with ThreadPoolExecutor(max_workers=n) as ex:
                parts = list(ex.map(DataUtilities._load_spec, specs))
        data, folders = [], []
        for spec, recs in zip(specs, parts):
            data.extend(recs)
            folders.extend([spec.get("data_folder", "") or ""] * len(recs))
        logger.info(f"loaded {len(data)} records from {len(specs)} source(s) ({'processes' if processes else 'threads'})")
        return data, folders

    @staticmethod
    def smart_nframes(total_frames: int, video_fps: float, fps: Optional[float] = None, nframes: Optional[int] = None,
                      min_frames: int = 4, max_frames: int = 768) -> int:
        """Number of frames to sample: either ``nframes`` or ``total/video_fps*fps`` clamped to
        [min_frames, max_frames] and rounded to a multiple of the temporal patch (2)."""
        def rnd(x):
            return max(FRAME_FACTOR, int(round(x / FRAME_FACTOR)) * FRAME_FACTOR)

        if nframes is not None:
            n = rnd(nframes)
        else:
            fps = fps or 2.0
            lo = math.ceil(min_frames / FRAME_FACTOR) * FRAME_FACTOR
            hi = max(lo, math.floor(min(max_frames, total_frames) / FRAME_FACTOR) * FRAME_FACTOR)
            n = total_frames / max(video_fps, 1e-6) * fps
            n = min(max(n, lo), hi)
            n = math.floor(n / FRAME_FACTOR) * FRAME_FACTOR
        return int(min(max(n, FRAME_FACTOR), max(total_frames, FRAME_FACTOR)))

    @staticmethod
    def download_blob_to_stream(fetch: Callable[[], bytes], retries: int = 5, backoff: float = 1.0) -> io.BytesIO:
        """Run ``fetch`` with exponential back-off; object-store clients are injected by the caller."""
        err = None
        for i in range(retries):
            try:
                return io.BytesIO(fetch())
            except Exception as e:  # pragma: no cover - network dependent
                err = e
                time.sleep(backoff * (2 ** i))
        raise RuntimeError(f"download failed after {retries} attempts: {err}")
