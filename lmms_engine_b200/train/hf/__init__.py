from .trainer import DLLMTrainer, Trainer, WanVideoTrainer

__all__ = ["Trainer", "DLLMTrainer", "WanVideoTrainer"]
