"""Write a starter training YAML with every default spelled out (reference:
tools/generate_config/generate_default_yaml.py:12-67).

``python -m lmms_engine_b200.tools.generate_default_yaml --output my.yaml
[--trainer_type fsdp2_trainer] [--dataset_type vision_iterable] [--model Qwen/Qwen2.5-7B]``"""
from __future__ import annotations

import argparse
import dataclasses

import yaml

from ..datasets.config import DatasetConfig
from ..train.config import TrainingArguments


def default_config(trainer_type: str, dataset_type: str, model: str) -> dict:
    targs = {f.name: (f.default if f.default is not dataclasses.MISSING else
                      (f.default_factory() if f.default_factory is not dataclasses.MISSING else None))
             for f in dataclasses.fields(TrainingArguments)}
    dcfg = {name: fld.default for name, fld in DatasetConfig.model_fields.items() if not fld.is_required()}
    dcfg.update(dataset_type=dataset_type, dataset_format="yaml", dataset_path="data.yaml", processor_config={
        "processor_name": model, "processor_type": "qwen2_5_vl" if "vision" in dataset_type else "pure_text"})
    return {"trainer_type": trainer_type, "dataset_config": dcfg,
            "model_config": {"load_from_pretrained_path": model, "attn_implementation": "flash_attention_2"},
            "trainer_args": targs}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--output", default="default_train.yaml")
    ap.add_argument("--trainer_type", default="fsdp2_trainer")
    ap.add_argument("--dataset_type", default="vision_iterable")
    ap.add_argument("--model", default="Qwen/Qwen2.5-VL-7B-Instruct")
    a = ap.parse_args(argv)
    cfg = default_config(a.trainer_type, a.dataset_type, a.model)
    with open(a.output, "w") as f:
        yaml.safe_dump(cfg, f, sort_keys=False)
    print(a.output)


if __name__ == "__main__":
    main()
