"""ShareGPT-style conversations (``{"id", "conversations": [{"from": "human" | "gpt", "value": ...}], "image" | "video" |
"audio": path}``) -> the ``messages`` schema of this engine, written as parquet (``id``, ``messages`` as a JSON string)
or jsonl.

``<image>`` / ``<video>`` / ``<audio>`` markers in a human turn become content items that point at the record's media
(a record with a ``video`` and an ``<image>`` marker - the LLaVA-Video-178K layout - becomes a ``video_url`` item); markers
beyond the media of a record are dropped with the text kept.  ``--system`` prepends a system message, e.g. the
"watch in silence, answer after the question" instruction of realtime question answering.  Inputs are JSON files (one
list per file) or jsonl; ``--glob`` patterns select them under ``--input-dir`` and ``--contains`` keeps files whose name
holds one of the given tags (the duration / task buckets of LLaVA-Video-178K: ``0_30_s``, ``_cap_``, ``_oe_``, ``_mc_``).

Plays the role of tools/convert_data/convert_llava_video_to_parquet.py of the reference for any dataset of this layout.

    python -m lmms_engine_b200.tools.convert_sharegpt --input-dir LLaVA-Video-178K --glob '0_30_s*/*_processed.json' \\
        --contains _cap_ _oe_ --output llava_video.parquet --system "You are a helpful video assistant. ..."
"""
from __future__ import annotations

import argparse
import glob
import json
import os
import re
from typing import Dict, Iterable, List, Optional

MARKERS = {"<image>": "image", "<video>": "video", "<audio>": "audio"}
KINDS = {"image": "image_url", "video": "video_url", "audio": "audio_url"}
ROLES = {"human": "user", "user": "user", "gpt": "assistant", "assistant": "assistant", "system": "system"}


def _media_of(entry: dict) -> Dict[str, List[str]]:
    out = {}
    for key in ("image", "video", "audio"):
        v = entry.get(key)
        out[key] = [v] if isinstance(v, str) else list(v or [])
    return out


def convert_entry(entry: dict, system: Optional[str] = None) -> dict:
    media = _media_of(entry)
    used = {k: 0 for k in media}
    messages: List[dict] = []
    if system:
        messages.append({"role": "system", "content": [{"type": "text", "text": system}]})
    for turn in entry["conversations"]:
        role = ROLES.get(turn.get("from", turn.get("role")))
        if role is None:
            raise ValueError(f"unknown speaker '{turn.get('from')}'")
        value = turn.get("value", turn.get("content", ""))
        content: List[dict] = []
        if role == "user":
            for piece in re.split(r"(<image>|<video>|<audio>)", value):
                kind = MARKERS.get(piece)
                if kind is None:
                    if piece.strip():
                        content.append({"type": "text", "text": piece.strip()})
                    continue
                # a record that only has a video answers an <image> marker with it
                pool = kind if used[kind] < len(media[kind]) else next((k for k in ("video", "image", "audio") if used[k] < len(media[k])), None)
                if pool is None:
                    continue
                url = media[pool][used[pool]]
                used[pool] += 1
                content.append({"type": KINDS[pool], KINDS[pool]: {"url": url}})
            content.sort(key=lambda c: c["type"] == "text")  # media first, then the text of the turn
            texts = [c for c in content if c["type"] == "text"]
            if len(texts) > 1:
                merged = {"type": "text", "text": "\n".join(c["text"] for c in texts)}
                content = [c for c in content if c["type"] != "text"] + [merged]
        else:
            content.append({"type": "text", "text": value})
        messages.append({"role": role, "content": content})
    return {"id": str(entry.get("id", "unknown")), "messages": messages}


def read_entries(path: str) -> Iterable[dict]:
    with open(path) as f:
        if path.endswith(".jsonl"):
            for line in f:
                if line.strip():
                    yield json.loads(line)
        else:
            yield from json.load(f)


def convert_files(paths: List[str], system: Optional[str] = None, max_per_file: int = 0) -> List[dict]:
    rows = []
    for p in paths:
        kept = 0
        for entry in read_entries(p):
            if max_per_file and kept >= max_per_file:
                break
            try:
                rows.append(convert_entry(entry, system))
                kept += 1
            except Exception as e:  # a damaged record does not end the conversion
                print(f"  skipping {entry.get('id', '?')} of {p}: {e}")
        print(f"{p}: {kept} rows")
    return rows


def write_rows(rows: List[dict], output: str) -> None:
    os.makedirs(os.path.dirname(os.path.abspath(output)), exist_ok=True)
    if output.endswith(".parquet"):
        import pyarrow as pa
        import pyarrow.parquet as pq

        pq.write_table(pa.table({"id": pa.array([r["id"] for r in rows], type=pa.string()),
                                 "messages": pa.array([json.dumps(r["messages"]) for r in rows], type=pa.string())}), output)
    else:
        with open(output, "w") as g:
            for r in rows:
                g.write(json.dumps(r) + "\n")


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--input", nargs="*", default=[], help="JSON / jsonl files")
    ap.add_argument("--input-dir", default=None)
    ap.add_argument("--glob", nargs="*", default=["*.json"], help="patterns under --input-dir")
    ap.add_argument("--contains", nargs="*", default=[], help="keep files whose name holds one of these tags")
    ap.add_argument("--system", default=None)
    ap.add_argument("--max-per-file", type=int, default=0)
    ap.add_argument("--output", required=True, help=".parquet or .jsonl")
    a = ap.parse_args(argv)
    paths = list(a.input)
    if a.input_dir:
        for pattern in a.glob:
            paths += sorted(glob.glob(os.path.join(a.input_dir, pattern)))
    if a.contains:
        paths = [p for p in paths if any(tag in os.path.basename(p) for tag in a.contains)]
    if not paths:
        raise SystemExit("no input files matched")
    rows = convert_files(paths, a.system, a.max_per_file)
    write_rows(rows, a.output)
    print(f"{len(rows)} rows -> {a.output}")


if __name__ == "__main__":
    main()
