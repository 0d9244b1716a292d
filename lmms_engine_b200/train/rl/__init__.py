from .grpo_trainer import GRPOTrainer, group_advantages, grpo_token_loss, register_reward
from .flow_grpo_trainer import FlowGRPOTrainer  # noqa: F401

__all__ = ["GRPOTrainer", "group_advantages", "grpo_token_loss", "register_reward"]
