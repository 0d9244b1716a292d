from .config import TrainerConfig, TrainingArguments
from .registry import TRAINER_REGISTER
from .fsdp2 import FSDP2SFTTrainer  # noqa: F401  (registers "fsdp2_trainer")
from .runner import TrainRunner

__all__ = ["TrainerConfig", "TrainingArguments", "TRAINER_REGISTER", "TrainRunner"]
