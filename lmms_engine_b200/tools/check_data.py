"""Dataset sanity check and token-length precompute (reference: tools/check_data/*).

Reads a json / jsonl / yaml(list of sources) dataset in the OpenAI-style ``messages`` schema, checks
that every referenced media file exists, estimates (or, with ``--processor``, measures) the token
length of each row and optionally writes the rows back with a ``precomputed_tokens`` field that the
packers use instead of their estimate.

``python -m lmms_engine_b200.tools.check_data --dataset data.yaml [--media_root DIR]
[--write out.jsonl] [--max_rows N]``"""
from __future__ import annotations

import argparse
import json
import os
from collections import Counter
from typing import Dict, Iterable, List

from ..utils.data_utils import DataUtilities

# per-item estimates used by the map-style dataset when no processor is run
EST = {"image_url": 2000, "audio_url": 750, "video_url": 5000}


def iter_media(row: dict) -> Iterable[tuple]:
    for m in row.get("messages", []):
        content = m.get("content")
        if isinstance(content, str):
            continue
        for part in content or []:
            t = part.get("type")
            if t in EST:
                v = part.get(t)
                yield t, (v.get("url") if isinstance(v, dict) else v)


def estimate_tokens(row: dict) -> int:
    n = 0
    for m in row.get("messages", []):
        content = m.get("content")
        if isinstance(content, str):
            n += int(len(content.split()) * 1.5)
            continue
        for part in content or []:
            t = part.get("type")
            n += EST.get(t, 0) if t in EST else int(len(str(part.get("text", "")).split()) * 1.5)
    return n


def check(rows: List[dict], media_root: str = "") -> Dict:
    missing, kinds, lengths = [], Counter(), []
    for i, row in enumerate(rows):
        for kind, url in iter_media(row):
            kinds[kind] += 1
            if url and "://" not in url and not os.path.exists(os.path.join(media_root, url)):
                missing.append((i, url))
        lengths.append(row.get("precomputed_tokens") or estimate_tokens(row))
    lengths_sorted = sorted(lengths)
    pct = lambda p: lengths_sorted[min(len(lengths_sorted) - 1, int(p * len(lengths_sorted)))] if lengths_sorted else 0
    return {"rows": len(rows), "media": dict(kinds), "missing": missing, "tokens_total": sum(lengths),
            "tokens_p50": pct(0.5), "tokens_p95": pct(0.95), "tokens_max": lengths_sorted[-1] if lengths_sorted else 0,
            "lengths": lengths}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--dataset", required=True)
    ap.add_argument("--format", default=None, choices=[None, "json", "jsonl", "yaml"])
    ap.add_argument("--media_root", default="")
    ap.add_argument("--write", default=None, help="write rows with precomputed_tokens to this jsonl")
    ap.add_argument("--max_rows", type=int, default=0)
    a = ap.parse_args(argv)
    fmt = a.format or os.path.splitext(a.dataset)[1].lstrip(".")
    rows = DataUtilities.load_yaml(a.dataset)[0] if fmt in ("yaml", "yml") else DataUtilities.load_one(a.dataset, fmt)
    if a.max_rows:
        rows = rows[: a.max_rows]
    rep = check(rows, a.media_root)
    lengths = rep.pop("lengths")
    print(json.dumps({**rep, "missing": rep["missing"][:20], "n_missing": len(rep["missing"])}, indent=1))
    if a.write:
        with open(a.write, "w") as f:
            for row, n in zip(rows, lengths):
                f.write(json.dumps({**row, "precomputed_tokens": n}) + "\n")
    return 1 if rep["missing"] else 0


if __name__ == "__main__":
    raise SystemExit(main())
