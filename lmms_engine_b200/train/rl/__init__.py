from .grpo_trainer import GRPOTrainer, group_advantages, grpo_token_loss, register_reward

__all__ = ["GRPOTrainer", "group_advantages", "grpo_token_loss", "register_reward"]
