from .config import TrainerConfig, TrainingArguments
from .registry import TRAINER_REGISTER
from .fsdp2 import FSDP2SFTTrainer  # noqa: F401  (registers "fsdp2_trainer")
from .fsdp2 import extra_trainers  # noqa: F401  (bagel / sit / rae trainers)
from . import hf, rl  # noqa: F401  (hf / dllm / wan / grpo trainers)
from .hf.trainer import DLLMTrainer, Trainer, WanVideoTrainer
from .runner import TrainRunner

__all__ = ["TrainerConfig", "TrainingArguments", "TRAINER_REGISTER", "TrainRunner", "FSDP2SFTTrainer", "Trainer", "DLLMTrainer",
           "WanVideoTrainer"]
