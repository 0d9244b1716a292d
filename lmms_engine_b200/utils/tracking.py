"""Experiment tracking: console always, wandb / tensorboard when asked for and importable
(reference: src/lmms_engine/utils/tracking.py:29-83, which only wires wandb)."""
from __future__ import annotations

import json
import os
from typing import Any, Dict, Iterable, Optional, Union

from .logging_utils import logger


class Tracking:
    supported_backend = ["wandb", "tensorboard", "console", "jsonl"]

    def __init__(self, project_name: Optional[str] = None, experiment_name: Optional[str] = None,
                 default_backend: Union[str, Iterable[str]] = "console", config: Optional[dict] = None,
                 output_dir: Optional[str] = None):
        if isinstance(default_backend, str):
            default_backend = [default_backend]
        self.backends: Dict[str, Any] = {}
        for b in default_backend:
            if b in ("none", None):
                continue
            if b == "all":
                b = "wandb"
            if b not in self.supported_backend:
                logger.warning(f"tracking backend '{b}' is not supported; ignoring")
                continue
            if b == "wandb":
                try:
                    import wandb

                    wandb.init(project=project_name or os.environ.get("WANDB_PROJECT", "lmms-engine"),
                               name=experiment_name or os.environ.get("WANDB_NAME"), config=config)
                    self.backends["wandb"] = wandb
                except Exception as e:  # offline boxes
                    logger.warning(f"wandb unavailable ({e}); falling back to console")
            elif b == "tensorboard":
                try:
                    from torch.utils.tensorboard import SummaryWriter

                    self.backends["tensorboard"] = SummaryWriter(os.path.join(output_dir or ".", "tb"))
                except Exception as e:
                    logger.warning(f"tensorboard unavailable ({e})")
            elif b == "jsonl":
                os.makedirs(output_dir or ".", exist_ok=True)
                self.backends["jsonl"] = open(os.path.join(output_dir or ".", "metrics.jsonl"), "a")
        self.backends.setdefault("console", True)

    def log(self, data: Dict[str, Any], step: int, backend: Optional[Iterable[str]] = None) -> None:
        for name, inst in self.backends.items():
            if backend is not None and name not in backend:
                continue
            if name == "wandb":
                inst.log(data=data, step=step)
            elif name == "tensorboard":
                for k, v in data.items():
                    if isinstance(v, (int, float)):
                        inst.add_scalar(k, v, step)
            elif name == "jsonl":
                inst.write(json.dumps({"step": step, **{k: v for k, v in data.items() if isinstance(v, (int, float, str))}}) + "\n")
                inst.flush()
            elif name == "console":
                parts = [f"{k}={v:.6g}" if isinstance(v, float) else f"{k}={v}" for k, v in data.items()]
                logger.info(f"step {step} | " + " ".join(parts))

    def finish(self) -> None:
        if "wandb" in self.backends:
            try:
                self.backends["wandb"].finish()
            except Exception:
                pass
        if "jsonl" in self.backends:
            self.backends["jsonl"].close()
