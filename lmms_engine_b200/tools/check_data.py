"""Dataset checks and token-length precompute (the reference keeps these as six scripts under ``tools/check_data``:
``check_dataset_yaml``, ``check_dataset_tokens``, ``precompute_tokens``, ``precompute_tokens_inline`` and the ``*_cloud``
variants of the last three; here they are subcommands of one tool sharing one media-measuring core).

Input: a YAML ``{datasets: [{path, data_folder, data_type}]}`` or a single json / jsonl file in the OpenAI-style
``messages`` schema.

``python -m lmms_engine_b200.tools.check_data exists  --dataset data.yaml [--out not_exists.txt]``
    every referenced media file exists (local folders or, with ``--object-storage``, blobs of a bucket).
``python -m lmms_engine_b200.tools.check_data tokens  --dataset data.yaml [--out tokens.txt]``
    estimated multimodal tokens per source (images by area, audio by duration, video by duration).
``python -m lmms_engine_b200.tools.check_data precompute --dataset data.yaml [--in-place | --out-dir DIR | --parquet FILE]``
    writes ``precomputed_tokens`` into every media (and text) part of every row, which the packers use instead of
    their flat estimates; ``--parquet`` writes one table of all sources (the "inline" form).
``python -m lmms_engine_b200.tools.check_data summary --dataset data.yaml``
    row counts, media counts, length percentiles (uses ``precomputed_tokens`` where present).

``--object-storage gcs|azure|local --bucket NAME`` reads media through the data plane's storage clients
(``utils/object_storage.py``) instead of the file system: the cloud variants.  ``--workers N`` sizes the thread pool
(media probing is I/O bound).  Unreadable media count with the reference's defaults (a 500 x 500 image, 30 s of audio,
32 frames of video) and are listed in the report.
"""
from __future__ import annotations

import argparse
import io
import json
import math
import os
import wave
from collections import Counter
from concurrent.futures import ThreadPoolExecutor
from typing import Dict, Iterable, List, Optional, Tuple

from ..utils.data_utils import DataUtilities

AUDIO_TOKENS_PER_SECOND = 25  # 750 tokens per 30 s
PATCH_AREA = 14 * 14 * 4  # pixels per token: 14 x 14 patches, 2 x 2 merged
VIDEO_TOKENS_PER_SECOND = (360 * 420) / PATCH_AREA  # one 360 x 420 frame per second of video
DEFAULTS = {"image_url": 500 * 500 // PATCH_AREA, "audio_url": 750, "video_url": 32 * VIDEO_TOKENS_PER_SECOND}
EST = {"image_url": 2000, "audio_url": 750, "video_url": 5000}  # flat estimates when nothing is measured
MEDIA = tuple(EST)


class MediaProbe:
    """Measures one media file; ``client`` (an object-storage client) replaces the file system when given."""

    def __init__(self, client=None):
        self.client = client
        self.failed: List[Tuple[str, str]] = []

    def _open(self, path: str):
        if self.client is None:
            return path
        from ..utils.object_storage import fetch_stream

        return fetch_stream(self.client, path)

    def exists(self, path: str) -> bool:
        if self.client is None:
            return os.path.exists(path)
        try:
            self.client.read(path)
            return True
        except Exception:  # noqa: BLE001 - SDKs raise their own hierarchies
            return False

    def image(self, path: str) -> float:
        from PIL import Image

        with Image.open(self._open(path)) as im:
            w, h = im.size
        return w * h // PATCH_AREA

    def audio(self, path: str) -> float:
        src = self._open(path)
        try:
            import soundfile as sf

            info = sf.info(src)
            seconds = info.frames / float(info.samplerate)
        except ImportError:
            with wave.open(src, "rb") as w:
                seconds = w.getnframes() / float(w.getframerate())
        return math.ceil(seconds * AUDIO_TOKENS_PER_SECOND)

    def video(self, path: str) -> float:
        if self.client is not None:
            from ..utils.object_storage import fetch_to_cache

            path = fetch_to_cache(self.client, path)
        try:
            import decord

            vr = decord.VideoReader(path)
            seconds = len(vr) / float(vr.get_avg_fps())
        except ImportError:
            import cv2

            cap = cv2.VideoCapture(path)
            if not cap.isOpened():
                raise FileNotFoundError(path)
            seconds = cap.get(cv2.CAP_PROP_FRAME_COUNT) / float(cap.get(cv2.CAP_PROP_FPS) or 25.0)
            cap.release()
        return seconds * VIDEO_TOKENS_PER_SECOND

    def tokens(self, kind: str, path: str) -> float:
        try:
            return {"image_url": self.image, "audio_url": self.audio, "video_url": self.video}[kind](path)
        except Exception as e:  # noqa: BLE001 - any unreadable file falls back to the default, and is reported
            self.failed.append((path, f"{type(e).__name__}: {e}"))
            return DEFAULTS[kind]


def iter_media(row: dict) -> Iterable[Tuple[str, dict]]:
    for m in row.get("messages", []):
        content = m.get("content")
        if isinstance(content, str):
            continue
        for part in content or []:
            if part.get("type") in MEDIA:
                yield part["type"], part


def media_url(kind: str, part: dict) -> Optional[str]:
    v = part.get(kind)
    return v.get("url") if isinstance(v, dict) else v


def estimate_tokens(row: dict) -> int:
    """Row length from ``precomputed_tokens`` where present, flat estimates otherwise."""
    n = 0.0
    for m in row.get("messages", []):
        content = m.get("content")
        if isinstance(content, str):
            n += len(content.split()) * 1.5
            continue
        for part in content or []:
            if "precomputed_tokens" in part:
                n += float(part["precomputed_tokens"])
            elif part.get("type") in MEDIA:
                n += EST[part["type"]]
            else:
                n += len(str(part.get("text", "")).split()) * 1.5
    return int(n)


def load_sources(path: str, fmt: Optional[str] = None) -> List[Dict]:
    """``[{path, data_folder, data_type, rows}]`` of a YAML of sources or of one file."""
    fmt = fmt or os.path.splitext(path)[1].lstrip(".")
    if fmt in ("yaml", "yml"):
        import yaml

        with open(path) as f:
            specs = yaml.safe_load(f)["datasets"]
    else:
        specs = [{"path": path, "data_folder": "", "data_type": fmt}]
    out = []
    for s in specs:
        kind = s.get("data_type", "json")
        out.append({"path": s["path"], "data_folder": s.get("data_folder") or "", "data_type": kind,
                    "rows": DataUtilities.load_one(s["path"], kind)})
    return out


def _pool(workers: int):
    return ThreadPoolExecutor(max_workers=max(1, workers))


# ---- subcommands ------------------------------------------------------------------------------------------------
def cmd_exists(sources, probe: MediaProbe, workers: int, out: Optional[str]) -> int:
    jobs = [(os.path.join(s["data_folder"], u) if probe.client is None else os.path.join(s["data_folder"], u).lstrip("/"))
            for s in sources for row in s["rows"] for k, p in iter_media(row) if (u := media_url(k, p)) and "://" not in u]
    with _pool(workers) as ex:
        found = list(ex.map(probe.exists, jobs))
    missing = [j for j, ok in zip(jobs, found) if not ok]
    print(json.dumps({"media": len(jobs), "missing": len(missing), "first": missing[:20]}, indent=1))
    if out:
        with open(out, "w") as f:
            f.writelines(m + "\n" for m in missing)
    return 1 if missing else 0


def _row_media_tokens(probe: MediaProbe, folder: str, row: dict, write: bool) -> float:
    total = 0.0
    for kind, part in iter_media(row):
        url = media_url(kind, part)
        n = probe.tokens(kind, os.path.join(folder, url)) if url else DEFAULTS[kind]
        if write:
            part["precomputed_tokens"] = n
        total += n
    if write:
        for m in row.get("messages", []):
            for part in (m["content"] if isinstance(m.get("content"), list) else []):
                if part.get("type") == "text":
                    part["precomputed_tokens"] = len(part.get("text", "").split(" ")) * 1.25
        row.setdefault("id", "Unknown_ID")
    return total


def cmd_tokens(sources, probe: MediaProbe, workers: int, out: Optional[str]) -> int:
    lines = []
    for s in sources:
        with _pool(workers) as ex:
            totals = list(ex.map(lambda r: _row_media_tokens(probe, s["data_folder"], r, False), s["rows"]))
        lines.append(f"Dataset {s['path']},\nEstimated total multimodal tokens: {sum(totals) / 1e6:.2f}M ({int(sum(totals))})\n")
        print(lines[-1])
    if out:
        with open(out, "w") as f:
            f.write("\n".join(lines))
    _report_failures(probe)
    return 0


def cmd_precompute(sources, probe: MediaProbe, workers: int, in_place: bool, out_dir: Optional[str], parquet: Optional[str]) -> int:
    for s in sources:
        with _pool(workers) as ex:
            list(ex.map(lambda r: _row_media_tokens(probe, s["data_folder"], r, True), s["rows"]))
    if parquet:
        import pyarrow as pa
        import pyarrow.parquet as pq

        rows = [{"id": str(r.get("id", "Unknown_ID")), "messages": json.dumps(r["messages"]), "data_folder": s["data_folder"]}
                for s in sources for r in s["rows"]]
        pq.write_table(pa.Table.from_pylist(rows), parquet)
    else:
        for s in sources:
            if in_place:
                target = s["path"]
            elif out_dir:
                os.makedirs(out_dir, exist_ok=True)
                target = os.path.join(out_dir, os.path.splitext(os.path.basename(s["path"]))[0] + ".jsonl")
            else:
                raise SystemExit("precompute needs --in-place, --out-dir or --parquet")
            tmp = target + ".tmp"
            with open(tmp, "w") as f:  # rows are rewritten as jsonl whatever the input was, like the reference
                for r in s["rows"]:
                    f.write(json.dumps({"id": r.get("id", "Unknown_ID"), "messages": r["messages"]}) + "\n")
            os.replace(tmp, target)
    _report_failures(probe)
    return 0


def cmd_summary(sources, media_root: str = "") -> int:
    kinds, lengths, missing = Counter(), [], []
    for s in sources:
        root = s["data_folder"] or media_root
        for i, row in enumerate(s["rows"]):
            for kind, part in iter_media(row):
                kinds[kind] += 1
                url = media_url(kind, part)
                if url and "://" not in url and not os.path.exists(os.path.join(root, url)):
                    missing.append((s["path"], i, url))
            lengths.append(row.get("precomputed_tokens") or estimate_tokens(row))
    srt = sorted(lengths)
    pct = lambda p: srt[min(len(srt) - 1, int(p * len(srt)))] if srt else 0  # noqa: E731
    print(json.dumps({"rows": len(lengths), "media": dict(kinds), "n_missing": len(missing), "missing": missing[:20],
                      "tokens_total": sum(lengths), "tokens_p50": pct(0.5), "tokens_p95": pct(0.95), "tokens_max": srt[-1] if srt else 0}, indent=1))
    return 1 if missing else 0


def _report_failures(probe: MediaProbe):
    if probe.failed:
        print(json.dumps({"unreadable_media": len(probe.failed), "first": probe.failed[:10]}, indent=1))


def check(rows: List[dict], media_root: str = "") -> Dict:
    """Programmatic form of ``summary`` for one list of rows."""
    missing, kinds, lengths = [], Counter(), []
    for i, row in enumerate(rows):
        for kind, part in iter_media(row):
            kinds[kind] += 1
            url = media_url(kind, part)
            if url and "://" not in url and not os.path.exists(os.path.join(media_root, url)):
                missing.append((i, url))
        lengths.append(row.get("precomputed_tokens") or estimate_tokens(row))
    srt = sorted(lengths)
    pct = lambda p: srt[min(len(srt) - 1, int(p * len(srt)))] if srt else 0  # noqa: E731
    return {"rows": len(rows), "media": dict(kinds), "missing": missing, "tokens_total": sum(lengths), "tokens_p50": pct(0.5),
            "tokens_p95": pct(0.95), "tokens_max": srt[-1] if srt else 0, "lengths": lengths}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("command", nargs="?", default="summary", choices=["exists", "tokens", "precompute", "summary"])
    ap.add_argument("--dataset", "--yaml-file", dest="dataset", required=True)
    ap.add_argument("--format", default=None, choices=[None, "json", "jsonl", "yaml"])
    ap.add_argument("--media_root", default="")
    ap.add_argument("--out", default=None)
    ap.add_argument("--in-place", action="store_true")
    ap.add_argument("--out-dir", default=None)
    ap.add_argument("--parquet", "--output-file", dest="parquet", default=None)
    ap.add_argument("--object-storage", default="none")
    ap.add_argument("--bucket", default=None)
    ap.add_argument("--workers", type=int, default=32)
    ap.add_argument("--max_rows", type=int, default=0)
    a = ap.parse_args(argv)
    sources = load_sources(a.dataset, a.format)
    if a.max_rows:
        for s in sources:
            s["rows"] = s["rows"][: a.max_rows]
    if a.media_root:
        for s in sources:
            s["data_folder"] = s["data_folder"] or a.media_root
    from ..utils.object_storage import make_client

    probe = MediaProbe(make_client(a.object_storage, a.bucket))
    if a.command == "exists":
        return cmd_exists(sources, probe, a.workers, a.out)
    if a.command == "tokens":
        return cmd_tokens(sources, probe, a.workers, a.out)
    if a.command == "precompute":
        return cmd_precompute(sources, probe, a.workers, a.in_place, a.out_dir, a.parquet)
    return cmd_summary(sources, a.media_root)


if __name__ == "__main__":
    raise SystemExit(main())
