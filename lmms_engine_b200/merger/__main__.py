"""``python -m lmms_engine.merger --checkpoint_path P [--output_path O] [--checkpoint_type
regular|ema] [--model_general_type T]`` (reference: src/lmms_engine/merger/__main__.py:15-79)."""
import argparse

from .fsdp2 import FSDP2Merger


def main(argv=None):
    ap = argparse.ArgumentParser(description="Merge FSDP2 checkpoint shards into HF safetensors")
    ap.add_argument("--checkpoint_path", required=True, help="checkpoint-N directory or an output_dir containing them")
    ap.add_argument("--output_path", default=None)
    ap.add_argument("--checkpoint_type", default="regular", choices=["regular", "ema"])
    ap.add_argument("--model_general_type", default=None, choices=[None, "causal_lm", "masked_lm", "image_text_to_text", "general"])
    args = ap.parse_args(argv)
    out = FSDP2Merger(args.checkpoint_path, args.output_path, args.checkpoint_type, args.model_general_type).merge()
    print(out)


if __name__ == "__main__":
    main()
