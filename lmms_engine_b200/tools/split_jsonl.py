"""Split a ``.jsonl`` file into N nearly equal pieces (``name_chunked_i.jsonl``), e.g. one per preprocessing worker
(reference: tools/create_data/split_jsonlines.py)."""
from __future__ import annotations

import argparse
from typing import List


def split(path: str, pieces: int) -> List[str]:
    with open(path) as f:
        lines = [l for l in f if l.strip()]
    size = (len(lines) + pieces - 1) // pieces
    stem = path[: -len(".jsonl")] if path.endswith(".jsonl") else path
    out = []
    for i in range(pieces):
        part = lines[i * size:(i + 1) * size]
        name = f"{stem}_chunked_{i}.jsonl"
        with open(name, "w") as f:
            f.writelines(part)
        out.append(name)
    return out


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--input", "-i", required=True)
    ap.add_argument("--num-split", "-s", type=int, required=True)
    args = ap.parse_args(argv)
    return split(args.input, args.num_split)


if __name__ == "__main__":
    main()
