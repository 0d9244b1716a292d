"""Step, memory-snapshot and CUDA-event profilers with the reference's config keys and
output file names (src/lmms_engine/utils/profiler.py:12-309)."""
from __future__ import annotations

import json
import os
from typing import Any, Dict, List, Optional, Tuple

import torch

from .logging_utils import logger


class StepProfiler:
    """torch.profiler over steps [start_step, end_step); Chrome trace under ``output_dir/profiler``."""

    def __init__(self, enable: bool, directory: str, profiler_config: Optional[Dict[str, Any]] = None, rank: int = 0):
        cfg = profiler_config or {}
        self.enable = bool(enable)
        self.start_step = int(cfg.get("start_step", 1))
        self.end_step = int(cfg.get("end_step", 3))
        self.rank = rank
        self.directory = os.path.join(directory, "profiler")
        self.prof = None
        if self.enable:
            acts = [torch.profiler.ProfilerActivity.CPU]
            if torch.cuda.is_available():
                acts.append(torch.profiler.ProfilerActivity.CUDA)
            self.prof = torch.profiler.profile(
                activities=acts,
                schedule=torch.profiler.schedule(wait=max(self.start_step, 0), warmup=1,
                                                 active=max(self.end_step - self.start_step, 1), repeat=1),
                record_shapes=True, profile_memory=True, with_stack=True,
            )
            self._saved = False

    def start(self):
        if self.prof is not None:
            self.prof.start()

    def step(self):
        if self.prof is not None:
            self.prof.step()

    def stop(self):
        if self.prof is not None:
            self.prof.stop()

    def stop_and_save(self):
        if self.prof is None or self._saved:
            return
        self.prof.stop()
        os.makedirs(self.directory, exist_ok=True)
        path = os.path.join(self.directory, f"prof_start_{self.start_step}_end_{self.end_step}_rank_{self.rank}.json")
        self.prof.export_chrome_trace(path)
        self._saved = True
        logger.info(f"profiler trace written to {path}")


class MemorySnapshotProfiler:
    """CUDA caching-allocator history; dumps a ``.pickle`` on demand, at ``stop_step`` or on OOM."""

    def __init__(self, enable: bool, directory: str, config: Optional[Dict[str, Any]] = None, rank: int = 0):
        cfg = config or {}
        self.enable = bool(enable) and torch.cuda.is_available()
        self.max_entries = int(cfg.get("max_entries", 100000))
        self.stop_step = cfg.get("stop_step")
        self.rank = rank
        self.directory = os.path.join(directory, "memory_snapshot")
        self.active = False

    def start(self):
        if not self.enable:
            return
        torch.cuda.memory._record_memory_history(max_entries=self.max_entries)
        self.active = True

    def step(self, step: int):
        if not self.active:
            return
        if torch.cuda.is_available():
            torch.cuda.nvtx.mark(f"step_{step}")
        if self.stop_step is not None and step >= int(self.stop_step):
            self.dump(f"step_{step}")
            self.stop()

    def dump(self, tag: str) -> Optional[str]:
        if not self.active:
            return None
        os.makedirs(self.directory, exist_ok=True)
        path = os.path.join(self.directory, f"memory_snapshot_{tag}_rank_{self.rank}.pickle")
        try:
            torch.cuda.memory._dump_snapshot(path)
            logger.info(f"memory snapshot written to {path}")
            return path
        except Exception as e:  # pragma: no cover
            logger.error(f"failed to dump memory snapshot: {e}")
            return None

    def dump_on_oom(self):
        return self.dump("oom")

    def stop(self):
        if self.active:
            torch.cuda.memory._record_memory_history(enabled=None)
            self.active = False


class CudaEventProfiler:
    """Named CUDA-event pairs around phases of a step; finished pairs are flushed without
    blocking (``event.query()``) into ``cuda_event_profiler/cuda_events_rank_{r}.jsonl``.

    Config: ``start_step`` (default 0), ``end_step`` (exclusive, default: never), ``stride``
    (record every n-th step), ``ranks`` (list, default all).
    """

    def __init__(self, enable: bool, directory: str, config: Optional[Dict[str, Any]] = None, rank: int = 0):
        cfg = config or {}
        self.rank = rank
        ranks = cfg.get("ranks")
        self.enable = bool(enable) and torch.cuda.is_available() and (ranks is None or rank in ranks)
        self.start_step = int(cfg.get("start_step", 0))
        self.end_step = cfg.get("end_step")
        self.stride = max(int(cfg.get("stride", 1)), 1)
        self.directory = os.path.join(directory, "cuda_event_profiler")
        self.path = os.path.join(self.directory, f"cuda_events_rank_{rank}.jsonl")
        self._open: Dict[str, Any] = {}
        self._pending: List[Tuple[int, str, Any, Any]] = []
        self._step = 0
        self._fh = None

    def _active(self) -> bool:
        if not self.enable or self._step < self.start_step:
            return False
        if self.end_step is not None and self._step >= int(self.end_step):
            return False
        return (self._step - self.start_step) % self.stride == 0

    def set_step(self, step: int) -> None:
        self._step = step

    def start(self, name: str) -> None:
        if not self._active():
            return
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        self._open[name] = ev

    def stop(self, name: str) -> None:
        ev0 = self._open.pop(name, None)
        if ev0 is None:
            return
        ev1 = torch.cuda.Event(enable_timing=True)
        ev1.record()
        self._pending.append((self._step, name, ev0, ev1))

    def flush(self, force: bool = False) -> None:
        if not self._pending:
            return
        keep = []
        for step, name, e0, e1 in self._pending:
            if force:
                e1.synchronize()
            if force or e1.query():
                if self._fh is None:
                    os.makedirs(self.directory, exist_ok=True)
                    self._fh = open(self.path, "a")
                self._fh.write(json.dumps({"step": step, "name": name, "rank": self.rank, "ms": e0.elapsed_time(e1)}) + "\n")
            else:
                keep.append((step, name, e0, e1))
        self._pending = keep
        if self._fh is not None:
            self._fh.flush()

    def close(self) -> None:
        self.flush(force=True)
        if self._fh is not None:
            self._fh.close()
            self._fh = None
