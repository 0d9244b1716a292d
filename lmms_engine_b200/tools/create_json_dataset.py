"""Turn (question, answer, media) records into the ``messages`` schema the datasets read
(reference: tools/create_json_dataset.py, tools/convert_data/*).

Input: jsonl with ``{"question", "answer", "image"|"video"|"audio": path-or-list}`` per line."""
from __future__ import annotations

import argparse
import json


def to_messages(rec: dict) -> dict:
    content = []
    for kind, key in (("image_url", "image"), ("video_url", "video"), ("audio_url", "audio")):
        v = rec.get(key)
        for item in ([v] if isinstance(v, str) else (v or [])):
            content.append({"type": kind, kind: {"url": item}})
    content.append({"type": "text", "text": rec["question"]})
    return {"id": rec.get("id"), "messages": [{"role": "user", "content": content},
                                              {"role": "assistant", "content": [{"type": "text", "text": rec["answer"]}]}]}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--input", required=True)
    ap.add_argument("--output", required=True)
    a = ap.parse_args(argv)
    with open(a.input) as f, open(a.output, "w") as g:
        for line in f:
            if line.strip():
                g.write(json.dumps(to_messages(json.loads(line))) + "\n")
    print(a.output)


if __name__ == "__main__":
    main()
