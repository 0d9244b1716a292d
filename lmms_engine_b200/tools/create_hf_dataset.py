"""LLaVA-style ``conversations`` records -> the OpenAI-style ``messages`` schema, saved as a dataset on disk.

    python -m lmms_engine_b200.tools.create_hf_dataset --input llava.json --output ./llava_messages [--format parquet]

Same conversion as the reference's tools/create_hf_dataset.py:23-43 (which then pushes to the hub; there is no
network here, so the result is written as ``jsonl`` or, when ``pyarrow`` is importable, ``parquet``).
"""
from __future__ import annotations

import argparse
import json
import os
from typing import Iterable, List


def llava_to_messages(conversations: List[dict]) -> List[dict]:
    messages = []
    for turn in conversations:
        if turn.get("from") == "human":
            content = []
            for tag, kind in (("<image>", "image_url"), ("<video>", "video_url"), ("<audio>", "audio_url")):
                for _ in range(turn["value"].count(tag)):
                    content.append({"type": kind, kind: {"url": tag}})
            text = turn["value"]
            for tag in ("<image>", "<video>", "<audio>"):
                text = text.replace(tag, "")
            content.append({"type": "text", "text": text.strip()})
            messages.append({"role": "user", "content": content})
        elif turn.get("from") == "gpt":
            messages.append({"role": "assistant", "content": [{"type": "text", "text": turn["value"]}]})
    return messages


def _records(path: str) -> Iterable[dict]:
    with open(path) as f:
        if path.endswith(".jsonl"):
            for line in f:
                if line.strip():
                    yield json.loads(line)
        else:
            yield from json.load(f)


def convert(path: str) -> List[dict]:
    out = []
    for rec in _records(path):
        row = {k: v for k, v in rec.items() if k != "conversations"}
        row["messages"] = llava_to_messages(rec.get("conversations", []))
        out.append(row)
    return out


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--input", required=True)
    ap.add_argument("--output", required=True)
    ap.add_argument("--format", choices=("jsonl", "parquet"), default="jsonl")
    args = ap.parse_args(argv)
    rows = convert(args.input)
    os.makedirs(args.output, exist_ok=True)
    if args.format == "parquet":
        import pyarrow as pa
        import pyarrow.parquet as pq

        pq.write_table(pa.Table.from_pylist([{**r, "messages": json.dumps(r["messages"])} for r in rows]),
                       os.path.join(args.output, "train.parquet"))
    else:
        with open(os.path.join(args.output, "train.jsonl"), "w") as f:
            for r in rows:
                f.write(json.dumps(r) + "\n")
    return len(rows)


if __name__ == "__main__":
    main()
