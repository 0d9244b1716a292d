"""Host-side failure detection.

* ``checkpoint_is_complete`` / ``latest_valid_checkpoint``: a checkpoint directory counts only if its
  completion marker exists and every rank file listed there is present with the recorded size, so a
  job that died while saving (or a truncated file) resumes from the previous checkpoint instead of
  crashing.  The reference resumes from whatever ``checkpoint-*`` sorts last
  (src/lmms_engine/train/runner.py:202-205).
* ``Heartbeat``: every rank publishes its step (and a wall-clock stamp) in the process group's
  key-value store between steps; before launching the next step a rank can ask whether any peer has
  fallen silent or reported an error, and raise ``PeerFailure`` on the host instead of entering a
  collective that would never complete.  Nothing here touches the GPU.
"""
from __future__ import annotations

import json
import os
import time
from typing import Dict, List, Optional

MARKER = "checkpoint_complete.json"


class PeerFailure(RuntimeError):
    pass


def write_completion_marker(ckpt_dir: str) -> None:
    """Record every file of the checkpoint with its size; written last, by one rank, after a barrier."""
    files: Dict[str, int] = {}
    for root, _, names in os.walk(ckpt_dir):
        for n in names:
            if n == MARKER:
                continue
            p = os.path.join(root, n)
            files[os.path.relpath(p, ckpt_dir)] = os.path.getsize(p)
    tmp = os.path.join(ckpt_dir, MARKER + ".tmp")
    with open(tmp, "w") as f:
        json.dump({"files": files, "time": time.time()}, f)
    os.replace(tmp, os.path.join(ckpt_dir, MARKER))


def checkpoint_is_complete(ckpt_dir: str) -> bool:
    marker = os.path.join(ckpt_dir, MARKER)
    if not os.path.exists(marker):
        return False
    try:
        rec = json.load(open(marker))
    except (OSError, ValueError):
        return False
    for rel, size in rec.get("files", {}).items():
        p = os.path.join(ckpt_dir, rel)
        if not os.path.exists(p) or os.path.getsize(p) != size:
            return False
    return True


def latest_valid_checkpoint(output_dir: str, candidates: List[str]) -> Optional[str]:
    """Newest complete checkpoint among ``candidates`` (sorted oldest to newest)."""
    for p in reversed(candidates):
        if checkpoint_is_complete(p):
            return p
    return None


class Heartbeat:
    """Step counter per rank in a c10d store (``TCPStore`` / ``FileStore`` / ``HashStore``)."""

    def __init__(self, store, rank: int, world: int, timeout_s: float = 60.0, prefix: str = "hb"):
        self.store, self.rank, self.world, self.timeout_s, self.prefix = store, rank, world, timeout_s, prefix

    def _key(self, r: int) -> str:
        return f"{self.prefix}/{r}"

    def beat(self, step: int) -> None:
        self.store.set(self._key(self.rank), json.dumps({"step": step, "t": time.time(), "error": None}))

    def report_error(self, step: int, message: str) -> None:
        self.store.set(self._key(self.rank), json.dumps({"step": step, "t": time.time(), "error": message[:500]}))

    def peer_state(self, r: int) -> Optional[dict]:
        try:
            if hasattr(self.store, "check") and not self.store.check([self._key(r)]):
                return None
            return json.loads(self.store.get(self._key(r)).decode())
        except (RuntimeError, ValueError):
            return None

    def check_peers(self, my_step: int) -> None:
        """Raise ``PeerFailure`` if a peer reported an error, or lags behind ``my_step`` and has not
        beaten for ``timeout_s``."""
        now = time.time()
        for r in range(self.world):
            if r == self.rank:
                continue
            st = self.peer_state(r)
            if st is None:
                continue  # has not started beating yet
            if st.get("error"):
                raise PeerFailure(f"rank {r} failed at step {st['step']}: {st['error']}")
            if st["step"] < my_step and now - st["t"] > self.timeout_s:
                raise PeerFailure(f"rank {r} has been silent for {now - st['t']:.1f}s at step {st['step']} (this rank is at {my_step})")

    def wait_for_peers(self, my_step: int, poll_s: float = 0.05) -> None:
        """Block (on the host) until every peer has reached ``my_step``, a peer fails, or the timeout runs out."""
        deadline = time.time() + self.timeout_s
        while True:
            behind = []
            for r in range(self.world):
                if r == self.rank:
                    continue
                st = self.peer_state(r)
                if st is not None and st.get("error"):
                    raise PeerFailure(f"rank {r} failed at step {st['step']}: {st['error']}")
                if st is None or st["step"] < my_step:
                    behind.append(r)
            if not behind:
                return
            if time.time() > deadline:
                raise PeerFailure(f"ranks {behind} did not reach step {my_step} within {self.timeout_s}s")
            time.sleep(poll_s)
