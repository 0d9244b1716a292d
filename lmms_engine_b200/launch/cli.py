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
from ..utils.config_loader import load_config
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
        logger.warning(f"trainer_args entries that this engine does not know are ignored: {sorted(dropped)}")
    return kept


def _init_distributed(raw_args: Dict[str, Any]) -> bool:
    """Bring up ``torch.distributed`` (env:// rendezvous; a lone process gets a local one) and the
    process-group manager for the degrees the trainer arguments ask for.  Returns ``use_cpu``."""
    from ..parallel.process_group_manager import RankLayout

    world = int(os.environ.get("WORLD_SIZE", "1"))
    # all mesh arithmetic and its error messages live in RankLayout; this builds the layout once up front so a
    # bad combination of degrees fails before any process group exists
    layout = RankLayout.from_degrees(world, tp=raw_args.get("tp_degree"), cp=raw_args.get("sp_ulysses_degree"),
                                     ep=raw_args.get("ep_degree"),
                                     hsdp_shard=(raw_args.get("fsdp_config") or {}).get("hsdp_shard_size"))
    cpu = bool(raw_args.get("use_cpu")) or not torch.cuda.is_available()
    if not dist.is_initialized():
        if world == 1 and "MASTER_ADDR" not in os.environ:
            os.environ.update(MASTER_ADDR="127.0.0.1", RANK="0", WORLD_SIZE="1", LOCAL_RANK="0")
            os.environ.setdefault("MASTER_PORT", "29500")
        if not cpu:
            torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        dist.init_process_group(backend="gloo" if cpu else "nccl", init_method="env://", world_size=world,
                                rank=int(os.environ.get("RANK", "0")),
                                timeout=datetime.timedelta(seconds=raw_args.get("ddp_timeout", 1800)))
    setup_process_group_manager(tp_size=layout.tp, cp_size=layout.cp, pp_size=1, dp_size=layout.dp, ep_size=layout.ep,
                                hsdp_shard_size=layout.hsdp_shard)
    return cpu


def create_train_task(config: Dict[str, Any]):
    """Public entry point (``lmms_engine.launch.cli.create_train_task`` of the reference,
    src/lmms_engine/launch/cli.py:24-94): a config dict with ``trainer_type``, ``dataset_config``,
    ``model_config`` and ``trainer_args`` becomes a ``TrainRunner``; distributed state is set up on the way."""
    from ..train.runner import TrainRunner

    raw_args = dict(config.get("trainer_args") or {})
    if raw_args.get("deepspeed"):
        raise ValueError(
            "trainer_args.deepspeed is set, but this engine has no DeepSpeed runtime: ZeRO-1/2 is what "
            "sharding_runtime: native does (optimizer state and gradients held by owner ranks), ZeRO-3 is "
            "sharding_runtime: native_sharded or torch_fsdp2.  Remove the deepspeed entry and pick one of those.")
    if _init_distributed(raw_args):
        raw_args["use_cpu"] = True
    if raw_args.get("eval_config") is not None:
        raw_args["eval_config"] = EvalConfig(**raw_args["eval_config"]).to_dict()
    train_config = TrainerConfig(
        dataset_config=DatasetConfig(**config["dataset_config"]),
        model_config=ModelConfig(**config["model_config"]),
        trainer_type=config["trainer_type"],
        trainer_args=TrainingArguments(**filter_training_args(raw_args)),
        extra_kwargs=config.get("extra_kwargs"),
    )
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
    defaults = deepcopy(config)
    config = ov.apply_overrides(config, rest)
    config_yaml = config.pop("config_yaml", None)
    if config_yaml:
        logger.info(f"config_yaml={config_yaml}: its entries are laid over the defaults, command-line overrides come last")
        loaded = load_config(config_yaml)  # .yaml / .yml / .json, also relative to the project root
        if isinstance(loaded, list):  # legacy form: a one-element list holding the config
            loaded = loaded[0]
            if "config" in loaded and "type" in loaded:
                loaded = loaded["config"]
        # the file replaces whole top-level sections of the defaults (as in the reference, src/lmms_engine/launch/cli.py:147-154);
        # the command line is then applied to the result, so `config_yaml=x.yaml trainer_args.max_steps=10` does what it says
        config = defaults
        config.update(loaded)
        config = ov.apply_overrides(config, rest)
        config.pop("config_yaml", None)
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
