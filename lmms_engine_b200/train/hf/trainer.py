"""``hf_trainer`` and its specialisations.

The reference subclasses ``transformers.Trainer`` (src/lmms_engine/train/hf/trainer.py:57-468);
``transformers.Trainer`` needs ``accelerate``, so here the same behaviour sits on the engine's own
loop:

* token-weighted loss: the number of supervised tokens of the step is summed over ranks
  (``get_batch_samples``, :238-290) and the loss is normalised by it
  (``average_tokens_across_devices``) instead of a mean of per-rank means;
* Muon parameter groups when ``use_muon`` (:377-468);
* checkpoints in the HF / accelerate FSDP2 layout: ``pytorch_model_fsdp_0`` holds
  ``torch.distributed.checkpoint`` (DCP) shards, next to ``trainer_state.json`` and
  ``rng_state_{rank}.pth``; ``only_save_mm_adapter`` writes ``mm_projector.bin`` (:304-332).

``dllm_trainer`` logs the masked-diffusion NLL next to the loss
(src/lmms_engine/train/hf/dllm_trainer.py:20-141); ``wan_trainer`` trains flow matching and
freezes the non-trainable towers (src/lmms_engine/train/hf/wan_trainer.py:15-96).
"""
from __future__ import annotations

import json
import os
import random
from typing import Any, Dict, Optional

import numpy as np
import torch
import torch.distributed as dist

from ...utils.logging_utils import logger
from ..fsdp2.fsdp2_trainer import FSDP2SFTTrainer
from ..registry import TRAINER_REGISTER
from .. import checkpoint as ckpt


@TRAINER_REGISTER.register("hf_trainer")
class Trainer(FSDP2SFTTrainer):
    def count_supervised_tokens(self, batch) -> torch.Tensor:
        n = (batch["labels"] != -100).sum().float() if "labels" in batch else torch.tensor(float(batch["input_ids"].numel()))
        n = n.to(self.device)
        if self.world_size > 1:
            dist.all_reduce(n, op=dist.ReduceOp.SUM)
        return n

    def compute_loss(self, batch, num_items_in_batch: Optional[torch.Tensor] = None):
        if not self.args.average_tokens_across_devices or not hasattr(self.model, "loss_reduction"):
            return super().compute_loss(batch)
        total = self.count_supervised_tokens(batch) if num_items_in_batch is None else num_items_in_batch
        prev = self.model.loss_reduction
        self.model.loss_reduction = "sum"
        try:
            loss = super().compute_loss(batch)
        finally:
            self.model.loss_reduction = prev
        # the data-parallel reduction averages over ranks: multiply back by the world size
        return loss * self.world_size / total.clamp(min=1.0)

    # ---- HF-layout checkpoints -------------------------------------------------------------
    def save_checkpoints(self, output_dir=None, step=None):
        if self.runtime_kind != "torch_fsdp2":
            path = super().save_checkpoints(output_dir, step)
        else:
            import torch.distributed.checkpoint as dcp

            step_ = self.global_step if step is None else step
            path = os.path.join(output_dir or self.args.output_dir, f"checkpoint-{step_}")
            os.makedirs(path, exist_ok=True)
            if getattr(self.args, "only_save_mm_adapter", False):
                self._save_mm_adapter(path)
            else:
                dcp.save({"model": self.model.state_dict()}, checkpoint_id=os.path.join(path, ckpt.MODEL_DIR))
                if not self.args.save_only_model:
                    dcp.save({"optimizer": self.optimizer.state_dict()}, checkpoint_id=os.path.join(path, "optimizer_0"))
            torch.save({"python": random.getstate(), "numpy": np.random.get_state(), "cpu": torch.get_rng_state(),
                        "cuda": torch.cuda.get_rng_state() if self.device.type == "cuda" else None},
                       os.path.join(path, f"rng_state_{self.rank}.pth"))
            if self.rank == 0:
                cfg = getattr(self.model, "config", None)
                if cfg is not None:
                    with open(os.path.join(path, "config.json"), "w") as f:
                        json.dump(cfg.to_dict(), f, indent=2, default=str)
                ckpt.rotate_checkpoints(output_dir or self.args.output_dir, self.args.save_total_limit)
            ckpt.barrier()
        if self.rank == 0:
            with open(os.path.join(path, "trainer_state.json"), "w") as f:
                json.dump({"global_step": self.global_step, "log_history": self.log_history[-200:],
                           "total_tokens": self.total_tokens}, f, indent=1)
        return path

    def load_checkpoints(self, path: str) -> None:
        marker = os.path.join(path, ckpt.MODEL_DIR, ".metadata")
        if self.runtime_kind == "torch_fsdp2" and os.path.exists(marker):
            import torch.distributed.checkpoint as dcp

            sd = {"model": self.model.state_dict()}
            dcp.load(sd, checkpoint_id=os.path.join(path, ckpt.MODEL_DIR))
            self.model.load_state_dict(sd["model"])
            opt_dir = os.path.join(path, "optimizer_0")
            if os.path.isdir(opt_dir):
                osd = {"optimizer": self.optimizer.state_dict()}
                dcp.load(osd, checkpoint_id=opt_dir)
                self.optimizer.load_state_dict(osd["optimizer"])
            ts = os.path.join(path, "trainer_state.json")
            if os.path.exists(ts):
                with open(ts) as f:
                    st = json.load(f)
                self.global_step, self.total_tokens = int(st["global_step"]), int(st.get("total_tokens", 0))
            return
        super().load_checkpoints(path)

    def _save_mm_adapter(self, path: str) -> None:
        keys = ("mm_projector", "merger", "audio_modal_projector", "vision_resampler")
        sd = {k: (v.full_tensor() if hasattr(v, "full_tensor") else v).cpu() for k, v in self.model.state_dict().items()
              if any(s in k for s in keys)}
        if self.rank == 0:
            torch.save(sd, os.path.join(path, "mm_projector.bin"))


@TRAINER_REGISTER.register("dllm_trainer")
class DLLMTrainer(Trainer):
    def calculate_training_metrics(self, seqlens, step_seconds):
        m = super().calculate_training_metrics(seqlens, step_seconds)
        nll = (self._last_out or {}).get("nll") if isinstance(self._last_out, dict) else None
        if nll is not None:
            v = nll.detach().float().clone()
            if self.world_size > 1:
                dist.all_reduce(v)
                v /= self.world_size
            m["train/nll"] = float(v)
        return m


@TRAINER_REGISTER.register("wan_trainer")
class WanVideoTrainer(Trainer):
    """Flow-matching training of the video diffusion family.  The model freezes everything outside
    ``config.trainable_modules`` itself (``freeze_except``); models without that method (a bare diffusion
    transformer) train whole."""

    def __init__(self, *a, **k):
        super().__init__(*a, **k)
        self.enable_perf_metrics = False

    def prepare_model(self):
        if hasattr(self.model, "freeze_except"):
            self.model.freeze_except()  # autoencoder / text / image encoders stay frozen and in eval mode
        super().prepare_model()
