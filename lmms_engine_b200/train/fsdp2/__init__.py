from .fsdp2_trainer import FSDP2SFTTrainer

__all__ = ["FSDP2SFTTrainer"]
