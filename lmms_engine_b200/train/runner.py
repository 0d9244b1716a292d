"""``TrainRunner``: build model / datasets / trainer from a ``TrainerConfig`` and run.

Mirrors the orchestration of the reference (src/lmms_engine/train/runner.py:37-264): seed,
sequence-parallel group, model from ``load_from_pretrained_path`` or ``load_from_config``
(+ ``overwrite_config``), datasets via the registry, trainer via ``TRAINER_REGISTER``,
``freeze_modules``, auto-resume from the newest ``checkpoint-*``.  There is no
monkey-patching stage: the native models already are the packed / fused implementation; the
``monkey_patch_kwargs`` of a config are accepted and mapped onto model switches.
"""
from __future__ import annotations

import os
import random
from typing import Any, Optional

import numpy as np
import torch

from ..mapping_func import DATASET_MAPPING, create_model_from_config, create_model_from_pretrained
from ..parallel import process_group_manager as pgm_mod
from ..parallel.sequence_parallel import ulysses
from ..utils.logging_utils import logger
from . import checkpoint as ckpt
from .config import TrainerConfig
from .registry import TRAINER_REGISTER


def set_seed(seed: int) -> None:
    random.seed(seed)
    np.random.seed(seed)
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)


class TrainRunner:
    def __init__(self, config: TrainerConfig) -> None:
        self.config = config
        self.train_dataset_config = config.dataset_config
        self.model_config = config.model_config
        self.model = None
        self.train_dataset = None
        self.eval_dataset = None
        self.trainer = None

    # ---- build ---------------------------------------------------------------------------
    def build(self):
        from .. import datasets as _ds  # noqa: F401
        from ..datasets import registry as _reg  # noqa: F401  (registers datasets / processors)

        set_seed(self.config.trainer_args.seed)
        self.create_sp_dis_group()
        self.model = self._build_model()
        self.train_dataset = self._build_train_dataset()
        if self.train_dataset_config.eval_dataset_path:
            self.eval_dataset = self._build_eval_dataset()
        self._apply_model_switches()
        self.trainer = self._build_trainer()
        return self

    def create_sp_dis_group(self):
        pgm = pgm_mod.process_group_manager
        if pgm is not None and pgm.cp_size > 1:
            ulysses.set_ulysses_sequence_parallel_group(pgm.cp_group)

    def _build_model(self):
        mc = self.model_config
        if mc.load_from_pretrained_path:
            model = create_model_from_pretrained(mc.load_from_pretrained_path, mc.model_general_type)
        elif mc.load_from_config:
            cfg = dict(mc.load_from_config)
            model_type = cfg.pop("model_type")
            conf = dict(cfg.pop("config", {}) or {})
            conf.update(mc.overwrite_config or {})
            args = self.config.trainer_args
            device = dtype = None
            if torch.cuda.is_available() and not args.use_cpu:
                # build straight on the GPU in the compute dtype
                device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
                dtype = torch.bfloat16 if args.bf16 else (torch.float16 if args.fp16 else None)
            model = create_model_from_config(model_type, conf, mc.model_general_type, device=device, dtype=dtype)
        else:
            raise ValueError("model_config needs load_from_pretrained_path or load_from_config")
        if mc.load_from_pretrained_path and mc.overwrite_config:
            for k, v in mc.overwrite_config.items():
                setattr(model.config, k, v)
        return model

    def _build_dataset(self, cfg):
        name = cfg.dataset_type
        if name not in DATASET_MAPPING:
            raise KeyError(f"dataset_type '{name}' is not registered; known: {sorted(DATASET_MAPPING)}")
        ds = DATASET_MAPPING[name](cfg)
        ds.build()
        return ds

    def _build_train_dataset(self):
        return self._build_dataset(self.train_dataset_config)

    def _build_eval_dataset(self):
        cfg = self.train_dataset_config.model_copy(update={"dataset_path": self.train_dataset_config.eval_dataset_path})
        return self._build_dataset(cfg)

    def _apply_model_switches(self):
        """Accept ``use_rmpad`` / ``use_liger_kernel`` / ``monkey_patch_kwargs``: they are always
        on in the native models; unknown switches are reported, never silently swallowed."""
        from ..models.monkey_patch import MONKEY_PATCHER

        kw = dict(self.model_config.monkey_patch_kwargs or {})
        model_type = getattr(getattr(self.model, "config", None), "model_type", None)
        if model_type is not None:
            # user-registered patches for this model type (none ship with the native models)
            MONKEY_PATCHER.apply(self.model, model_type, kw.get("patch_type", ["liger"]),
                                 **{k: v for k, v in kw.items() if k != "patch_type"})
        known = {"patch_type", "rope", "cross_entropy", "fused_linear_cross_entropy", "rms_norm", "swiglu", "use_rmpad"}
        extra = {k: v for k, v in kw.items() if k not in known}
        for k, v in extra.items():
            if hasattr(self.model, k):
                setattr(self.model, k, v)
            else:
                logger.warning(f"monkey_patch_kwargs.{k} has no counterpart in the native model and is ignored")

    def _build_trainer(self):
        cls = TRAINER_REGISTER[self.config.trainer_type]
        collator = self.train_dataset.get_collator()
        return cls(model=self.model, args=self.config.trainer_args, data_collator=collator,
                   train_dataset=self.train_dataset, eval_dataset=self.eval_dataset,
                   processing_class=getattr(self.train_dataset, "processor", None))

    # ---- run -----------------------------------------------------------------------------
    def freeze_modules(self):
        names = self.config.trainer_args.freeze_modules or []
        for modname in names:
            hit = False
            for n, m in self.model.named_modules():
                if n == modname or n.endswith("." + modname):
                    for p in m.parameters():
                        p.requires_grad_(False)
                    hit = True
            if not hit:
                logger.warning(f"freeze_modules: no module named '{modname}'")

    def run(self, **kwargs):
        args = self.config.trainer_args
        self.freeze_modules()
        resume = kwargs.get("resume_from_checkpoint") or args.resume_from_checkpoint
        if resume is None or resume is True:
            latest = ckpt.latest_resumable_checkpoint(args.output_dir)
            newest = ckpt.latest_checkpoint(args.output_dir)
            if newest is not None and latest != newest:
                logger.warning(f"{newest} is incomplete or damaged; resuming from {latest}")
            resume = latest if latest is not None else None
        result = self.trainer.train(resume_from_checkpoint=resume)
        return result
