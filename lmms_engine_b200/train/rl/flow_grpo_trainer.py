"""``flow_grpo_trainer``: group-relative policy optimisation of IMAGE generation for the unified (Bagel) model.

The reference keeps this as a loss inside the model driven by an external loop
(src/lmms_engine/models/bagel/bagel.py:885-1273: ``generate_image`` records the stochastic sampling steps,
``generate_image_learn`` replays them under the current policy; src/lmms_engine/models/bagel/inferencer.py:150-200 is
the only caller).  Here the loop is a registered trainer: for every prompt of the batch the policy samples a group of
images (latents) with SDE steps inside a window of the schedule, a registered reward scores each image, rewards are
normalised inside the group, and every recorded step contributes the clipped-ratio loss (plus a Gaussian KL to a frozen
copy when ``beta > 0``).  Like the reference, the optimizer moves after every recorded step.

``trainer_args.rl_config``: ``group_size`` (4), ``image_hw`` (latent patch grid, e.g. ``[16, 16]``), ``num_timesteps`` (24),
``sde_window`` (``[first, count]``; default all steps), ``noise_level`` (0.7), ``cfg_text_scale`` (1.0),
``clip_range`` (1e-4, or ``[lt, gt]``), ``beta`` (0.0), ``adv_clip_max`` (5.0), ``reward`` (registered name or
``module:function`` taking ``(prompt_ids, latent [C, H, W])``), ``boi_token_id`` / ``eoi_token_id``, ``uncond_ids``.
"""
from __future__ import annotations

import copy
from typing import Callable, Dict, List

import torch

from ..registry import TRAINER_REGISTER
from .grpo_trainer import GRPOTrainer, group_advantages, register_reward, resolve_reward


@register_reward("latent_brightness")
def _reward_brightness(prompt: torch.Tensor, latent: torch.Tensor) -> float:
    """Toy reward for tests and smoke runs: brighter first channel is better."""
    return float(latent[0].mean())


@TRAINER_REGISTER.register("flow_grpo_trainer")
class FlowGRPOTrainer(GRPOTrainer):
    def __init__(self, *a, **k):
        super().__init__(*a, **k)
        cfg = dict(self.args.rl_config or {})
        self.group_size = int(cfg.get("group_size", 4))
        self.image_hw = tuple(cfg.get("image_hw", (16, 16)))
        self.num_timesteps = int(cfg.get("num_timesteps", 24))
        self.sde_window = tuple(cfg["sde_window"]) if cfg.get("sde_window") else None
        self.noise_level = float(cfg.get("noise_level", 0.7))
        self.cfg_text_scale = float(cfg.get("cfg_text_scale", 1.0))
        clip = cfg.get("clip_range", 1e-4)
        self.clip = (float(clip), float(clip)) if not isinstance(clip, (list, tuple)) else (float(clip[0]), float(clip[1]))
        self.beta = float(cfg.get("beta", 0.0))
        self.adv_clip_max = float(cfg.get("adv_clip_max", 5.0))
        self.boi, self.eoi = int(cfg.get("boi_token_id", 0)), int(cfg.get("eoi_token_id", 0))
        self.uncond_ids = cfg.get("uncond_ids")
        self.reward_fn: Callable = resolve_reward(cfg.get("reward", "latent_brightness"))

    def resolve_runtime(self) -> str:
        # the policy pass steps the optimizer inside the model's replay loop: plain parameters on every rank
        return "torch_fsdp2" if self.world_size > 1 else "plain"

    def prepare_model(self):
        if self.world_size > 1:
            super().prepare_model()
        else:
            self.runtime_kind = "plain"
            self.model.to(self.device)
            if self.beta > 0:
                self.ref_model = copy.deepcopy(self.model).requires_grad_(False).eval()

    def prepare_optimizer(self):
        a = self.args
        params = [p for p in self.model.parameters() if p.requires_grad]
        self.optimizer = torch.optim.AdamW(params, lr=a.learning_rate, betas=(a.adam_beta1, a.adam_beta2), eps=a.adam_epsilon,
                                           weight_decay=a.weight_decay)
        for g in self.optimizer.param_groups:
            g.setdefault("initial_lr", g["lr"])

    def training_step(self, batch, do_step):
        model = self.model
        prompts = self.prompts_of(batch)
        uncond = torch.as_tensor(self.uncond_ids, device=self.device) if self.uncond_ids is not None else None
        model.eval()
        rollouts, rewards = [], []
        for p in prompts:
            for _ in range(self.group_size):
                r = model.generate_image(p, self.image_hw, self.boi, self.eoi, num_timesteps=self.num_timesteps, noise_level=self.noise_level,
                                         sde_window=self.sde_window, uncond_ids=uncond, cfg_text_scale=self.cfg_text_scale)
                rollouts.append(r)
                rewards.append(self.reward_fn(p, model.unpatchify_latent(r["image_latent"], self.image_hw)))
        rewards_t = torch.tensor(rewards, dtype=torch.float32, device=self.device)
        adv = group_advantages(rewards_t, self.group_size)
        model.train()
        self.lr_factor = self.current_lr_factor(self.global_step)
        for g in self.optimizer.param_groups:
            g["lr"] = g["initial_lr"] * self.lr_factor
        norms: List[torch.Tensor] = []

        def step(loss):
            loss.backward()
            norms.append(torch.nn.utils.clip_grad_norm_([p for g in self.optimizer.param_groups for p in g["params"]], self.args.max_grad_norm))
            self.optimizer.step()
            self.optimizer.zero_grad(set_to_none=True)

        stats: Dict[str, List[torch.Tensor]] = {}
        for r, a in zip(rollouts, adv):
            if not r["latents"]:
                continue
            out = model.grpo_learn(r, a, clip_range=self.clip, beta=self.beta, ref_model=self.ref_model, noise_level=self.noise_level,
                                   cfg_text_scale=self.cfg_text_scale, adv_clip_max=self.adv_clip_max, step_callback=step)
            for k_, v in out.items():
                stats.setdefault(k_, []).append(v)
        mean = {k_: float(torch.stack(v).mean()) for k_, v in stats.items()}
        self.rl_metrics = {"rl/reward_mean": float(rewards_t.mean()), "rl/reward_std": float(rewards_t.std(unbiased=False)),
                           "rl/policy_loss": mean.get("policy_loss", 0.0), "rl/kl": mean.get("kl_loss", 0.0),
                           "rl/clipfrac": mean.get("clipfrac", 0.0), "rl/recorded_steps": float(sum(len(r["latents"]) for r in rollouts))}
        loss = torch.tensor(mean.get("loss", 0.0), device=self.device)
        return loss, (torch.stack(norms).mean() if norms else None)
