"""Asynchronous evaluation through an lmms-eval HTTP server (reference:
src/lmms_engine/eval/backends.py:10-257): rank 0 submits a checkpoint as a job, a daemon thread
polls for completion, finished jobs are turned into ``eval/<task>_<metric>`` values that the
trainer logs against the training step that produced the checkpoint.  Failures are logged and
dropped; they never stop training."""
from __future__ import annotations

import json
import queue
import threading
import time
import urllib.error
import urllib.request
from typing import Any, Dict, Iterator, List, Optional, Tuple

from ..utils.logging_utils import logger


class EvalClient:
    """Minimal JSON-over-HTTP client: ``POST /evaluate`` -> ``{"job_id"}``, ``GET /jobs/<id>``."""

    def __init__(self, url: str, timeout: float = 30.0):
        self.url, self.timeout = url.rstrip("/"), timeout

    def _request(self, method: str, path: str, payload: Optional[dict] = None) -> dict:
        data = json.dumps(payload).encode() if payload is not None else None
        req = urllib.request.Request(self.url + path, data=data, method=method, headers={"Content-Type": "application/json"})
        with urllib.request.urlopen(req, timeout=self.timeout) as resp:
            return json.loads(resp.read().decode() or "{}")

    def submit(self, payload: dict) -> str:
        return str(self._request("POST", "/evaluate", payload)["job_id"])

    def status(self, job_id: str) -> dict:
        return self._request("GET", f"/jobs/{job_id}")


class EvalServerBackend:
    def __init__(self, eval_config: Dict[str, Any], output_dir: str = ".", client: Optional[EvalClient] = None):
        self.cfg = dict(eval_config)
        self.client = client or EvalClient(self.cfg.get("server_url", "http://localhost:8000"))
        self.poll_interval = float(self.cfg.get("poll_interval", 20.0))
        self.output_dir = output_dir
        self._jobs: Dict[str, int] = {}
        self._results: "queue.Queue[Tuple[int, Dict[str, float]]]" = queue.Queue()
        self._lock = threading.Lock()
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._poll_loop, daemon=True)
        self._thread.start()

    def build_payload(self, checkpoint_path: str) -> dict:
        c = self.cfg
        model_args = dict(c.get("model_args") or {})
        model_args[c.get("checkpoint_key", "model")] = checkpoint_path
        keys = ("model", "tasks", "num_fewshot", "batch_size", "device", "limit", "gen_kwargs", "log_samples", "predict_only", "num_gpus")
        payload = {k: c.get(k) for k in keys if c.get(k) is not None}
        payload["model_args"] = model_args
        return payload

    def submit(self, checkpoint_path: str, step: int) -> Optional[str]:
        try:
            job = self.client.submit(self.build_payload(checkpoint_path))
        except (urllib.error.URLError, OSError, KeyError, ValueError) as e:
            logger.warning(f"eval submit failed for step {step}: {e}")
            return None
        with self._lock:
            self._jobs[job] = step
        logger.info(f"submitted eval job {job} for step {step}")
        return job

    @staticmethod
    def parse_results(result: dict) -> Dict[str, float]:
        out: Dict[str, float] = {}
        for task, metrics in (result.get("results") or {}).items():
            for name, val in (metrics or {}).items():
                key = name.split(",")[0]
                if isinstance(val, (int, float)) and not isinstance(val, bool) and not key.endswith("_stderr"):
                    out[f"eval/{task}_{key}"] = float(val)
        return out

    def _poll_loop(self):
        while not self._stop.wait(self.poll_interval):
            with self._lock:
                jobs = dict(self._jobs)
            for job, step in jobs.items():
                try:
                    st = self.client.status(job)
                except (urllib.error.URLError, OSError, ValueError) as e:
                    logger.warning(f"eval poll failed for job {job}: {e}")
                    continue
                state = str(st.get("status", "")).lower()
                if state in ("completed", "finished", "done"):
                    self._results.put((step, self.parse_results(st.get("result") or st)))
                elif state in ("failed", "error", "cancelled"):
                    logger.warning(f"eval job {job} (step {step}) ended as {state}: {st.get('error')}")
                else:
                    continue
                with self._lock:
                    self._jobs.pop(job, None)

    def poll_results(self) -> Iterator[Tuple[int, Dict[str, float]]]:
        while True:
            try:
                yield self._results.get_nowait()
            except queue.Empty:
                return

    def pending(self) -> int:
        with self._lock:
            return len(self._jobs)

    def close(self):
        self._stop.set()
