"""Command-line entry point: ``python -m lmms_engine.launch.cli config_yaml=PATH [overrides]``.

Same three ways to configure a run as the reference (src/lmms_engine/launch/cli.py:141-161):
dotted overrides over the bundled ``default_config.yaml``, ``--config-path/--config-name``,
or the legacy ``config_yaml=`` file whose top-level keys replace the defaults wholesale.
``create_train_task(config_dict)`` is the programmatic entry used by tests.
"""
from __future__ import annotations

import datetime
import os
import shutil
import sys
from copy import deepcopy
from typing import Any, Dict, List, Optional

import torch
import torch.distributed as dist
import yaml

from ..datasets.config import DatasetConfig
from ..eval.config import EvalConfig
from ..models.config import ModelConfig
from ..parallel.process_group_manager import setup_process_group_manager
from ..train.config import TrainerConfig, TrainingArguments
from ..utils.logging_utils import logger, setup_distributed_logging
from . import overrides as ov

DEFAULT_CONFIG = os.path.join(os.path.dirname(__file__), "config", "default_config.yaml")


def filter_training_args(kwargs: Dict[str, Any]) -> Dict[str, Any]:
    valid = TrainingArguments.field_names()
    kept, dropped = {}, []
    for k, v in kwargs.items():
        if k in valid:
            kept[k] = v
        else:
            dropped.append(k)
    if dropped:
        logger.warning(f"Filtering out unsupported TrainingArguments parameters: {dropped}")
    return kept


def create_train_task(config: Dict[str, Any]):
    from ..train.runner import TrainRunner

    dataset_config = DatasetConfig(**config.pop("dataset_config"))
    model_config = ModelConfig(**config.pop("model_config"))
    trainer_type = config.pop("trainer_type")
    global_rank = int(os.environ.get("RANK", "0"))
    world_size = int(os.environ.get("WORLD_SIZE", "1"))

    trainer_args = config.get("trainer_args") or {}
    sp_degree = trainer_args.get("sp_ulysses_degree", 1) or 1
    tp_degree = trainer_args.get("tp_degree", 1) or 1
    ep_degree = trainer_args.get("ep_degree", 1) or 1
    if tp_degree < 1:
        raise ValueError(f"tp_degree must be >= 1, got {tp_degree}")
    if world_size % (sp_degree * tp_degree) != 0:
        raise ValueError(
            f"World size ({world_size}) must be divisible by sp_ulysses_degree ({sp_degree}) * tp_degree ({tp_degree})"
        )
    dp_size = world_size // (sp_degree * tp_degree)
    use_cpu = bool(trainer_args.get("use_cpu", False)) or not torch.cuda.is_available()
    backend = "gloo" if use_cpu else "nccl"
    ddp_timeout = trainer_args.get("ddp_timeout", 30 * 60)
    if not dist.is_initialized():
        if world_size == 1 and "MASTER_ADDR" not in os.environ:
            os.environ["MASTER_ADDR"] = "127.0.0.1"
            os.environ.setdefault("MASTER_PORT", "29500")
            os.environ["RANK"] = "0"
            os.environ["WORLD_SIZE"] = "1"
            os.environ["LOCAL_RANK"] = "0"
        if backend == "nccl":
            torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        dist.init_process_group(rank=global_rank, world_size=world_size, backend=backend, init_method="env://",
                                timeout=datetime.timedelta(seconds=ddp_timeout))
    fsdp_config = trainer_args.get("fsdp_config", {}) or {}
    hsdp_shard_size = fsdp_config.get("hsdp_shard_size", 0) or 0
    setup_process_group_manager(tp_size=tp_degree, cp_size=sp_degree, pp_size=1, dp_size=dp_size, ep_size=ep_degree,
                                hsdp_shard_size=hsdp_shard_size)
    trainer_args = dict(config.pop("trainer_args"))
    if use_cpu:
        trainer_args["use_cpu"] = True
    eval_cfg = trainer_args.pop("eval_config", None)
    if eval_cfg is not None:
        trainer_args["eval_config"] = EvalConfig(**eval_cfg).to_dict()
    args = TrainingArguments(**filter_training_args(trainer_args))
    train_config = TrainerConfig(dataset_config=dataset_config, model_config=model_config, trainer_type=trainer_type,
                                 trainer_args=args, extra_kwargs=config.get("extra_kwargs"))
    return TrainRunner(config=train_config)


def save_config(config: Dict[str, Any]) -> None:
    rank = int(os.environ.get("LOCAL_RANK", "0")) if dist.is_initialized() else 0
    if rank == 0:
        data_config = config.get("dataset_config") or {}
        output_dir = (config.get("trainer_args") or {}).get("output_dir", "./output")
        os.makedirs(output_dir, exist_ok=True)
        if data_config.get("dataset_format") == "yaml" and data_config.get("dataset_path"):
            shutil.copy(data_config["dataset_path"], os.path.join(output_dir, "dataset.yaml"))
        with open(os.path.join(output_dir, "config.yaml"), "w") as f:
            yaml.dump(config, f, default_flow_style=False, sort_keys=False)
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.barrier()


def build_config(argv: List[str]) -> Dict[str, Any]:
    cp, cn, rest = ov.split_argv(argv)
    config = ov.load_config_file(cp, cn, DEFAULT_CONFIG)
    config = ov.apply_overrides(config, rest)
    config_yaml = config.pop("config_yaml", None)
    if config_yaml:
        logger.info(f"Detected config yaml, merging with the default config. Will use the args in {config_yaml} to override current config.")
        with open(config_yaml) as f:
            loaded = yaml.safe_load(f)
        if isinstance(loaded, list):  # legacy form: a one-element list holding the config
            loaded = loaded[0]
            if "config" in loaded and "type" in loaded:
                loaded = loaded["config"]
        config.update(loaded)
    return config


def main(argv: Optional[List[str]] = None) -> None:
    setup_distributed_logging()
    config = build_config(list(sys.argv[1:] if argv is None else argv))
    original = deepcopy(config)
    task = create_train_task(config)
    save_config(original)
    task.build()
    task.run()
    if dist.is_initialized():
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
