"""Cumulative compute, energy and CO2 accounting written to ``compute_summary.json``
(reference: src/lmms_engine/utils/compute_tracker.py:25-130; energy = gpus * TDP * hours)."""
from __future__ import annotations

import json
import os
import time
from typing import Any, Dict

from .train_utils import TrainUtilities


class ComputeTracker:
    def __init__(self, num_gpus: int = 1, carbon_intensity: float = 0.475):
        self.num_gpus = num_gpus
        self.carbon_intensity = carbon_intensity
        self.total_flops = 0.0
        self.total_tokens = 0
        self.total_seconds = 0.0
        self.steps = 0
        self._tdp = TrainUtilities.get_device_tdp()

    def update(self, flops: float, tokens: int, seconds: float) -> None:
        self.total_flops += float(flops)
        self.total_tokens += int(tokens)
        self.total_seconds += float(seconds)
        self.steps += 1

    @property
    def energy_kwh(self) -> float:
        return self.num_gpus * self._tdp * (self.total_seconds / 3600.0) / 1000.0

    @property
    def co2_kg(self) -> float:
        return self.energy_kwh * self.carbon_intensity

    def summary(self) -> Dict[str, Any]:
        return {
            "total_flops": self.total_flops,
            "total_flops_human": TrainUtilities.format_flops(self.total_flops),
            "total_tokens": self.total_tokens,
            "total_tokens_human": TrainUtilities.format_tokens(self.total_tokens),
            "train_seconds": self.total_seconds,
            "gpu_hours": self.num_gpus * self.total_seconds / 3600.0,
            "num_gpus": self.num_gpus,
            "device_tdp_w": self._tdp,
            "energy_kwh": self.energy_kwh,
            "carbon_intensity_kg_per_kwh": self.carbon_intensity,
            "co2_kg": self.co2_kg,
            "steps": self.steps,
        }

    def state_dict(self) -> Dict[str, Any]:
        return {"total_flops": self.total_flops, "total_tokens": self.total_tokens, "total_seconds": self.total_seconds,
                "steps": self.steps}

    def load_state_dict(self, sd: Dict[str, Any]) -> None:
        self.total_flops = sd.get("total_flops", 0.0)
        self.total_tokens = sd.get("total_tokens", 0)
        self.total_seconds = sd.get("total_seconds", 0.0)
        self.steps = sd.get("steps", 0)

    def save(self, output_dir: str) -> str:
        os.makedirs(output_dir, exist_ok=True)
        path = os.path.join(output_dir, "compute_summary.json")
        with open(path, "w") as f:
            json.dump(self.summary(), f, indent=2)
        return path
