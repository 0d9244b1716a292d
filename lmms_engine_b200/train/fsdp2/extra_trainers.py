"""Trainer variants on the fsdp2 loop:

* ``bagel_fsdp2_trainer`` logs the cross-entropy and MSE parts (raw and weighted) and their
  token counts (reference: src/lmms_engine/train/fsdp2/bagel_fsdp2_trainer.py:31-167);
* ``sit_trainer`` keeps a full EMA copy of the model, updated every step and saved as ``ema.pt``;
  throughput metrics are off (reference: src/lmms_engine/train/fsdp2/sit_trainer.py:26-87);
* ``rae_trainer`` is the GAN recipe: a generator step with L1 (+ perceptual when weights are
  given) + adversarial loss whose weight is adapted from the gradient norms at the decoder's
  last layer, then discriminator step(s) with their own AdamW and schedule, differentiable
  augmentation, EMA saved as ``ema_state.pt`` (reference: src/lmms_engine/train/fsdp2/rae_trainer.py:22-480).
"""
from __future__ import annotations

import copy
import os
from typing import Any, Dict

import torch
import torch.distributed as dist
import torch.nn.functional as F

from ...utils import schedulers
from ...utils.logging_utils import logger
from ..registry import TRAINER_REGISTER
from .fsdp2_trainer import FSDP2SFTTrainer


@TRAINER_REGISTER.register("bagel_fsdp2_trainer")
class BagelFSDP2Trainer(FSDP2SFTTrainer):
    def compute_loss(self, batch):
        loss = super().compute_loss(batch)
        out = self._last_out
        self._parts = {k: out.get(k) for k in ("ce", "mse")}
        return loss

    def calculate_training_metrics(self, seqlens, step_seconds):
        m = super().calculate_training_metrics(seqlens, step_seconds)
        cfg = getattr(self.model, "config", None)
        for k, wname in (("ce", "ce_weight"), ("mse", "mse_weight")):
            v = getattr(self, "_parts", {}).get(k)
            if v is None:
                continue
            v = v.detach().float().clone()
            if self.world_size > 1:
                dist.all_reduce(v, op=dist.ReduceOp.SUM)
                v /= self.world_size
            m[f"train/{k}"] = float(v)
            m[f"train/{k}_weighted"] = float(v) * float(getattr(cfg, wname, 1.0))
        return m


@TRAINER_REGISTER.register("sit_trainer")
class SitTrainer(FSDP2SFTTrainer):
    def __init__(self, *a, **k):
        super().__init__(*a, **k)
        self.enable_perf_metrics = False
        self.ema_model = None

    def prepare_model(self):
        super().prepare_model()
        self.ema_model = copy.deepcopy(self.model).requires_grad_(False).eval()

    def training_step(self, batch, do_step):
        out = super().training_step(batch, do_step)
        if do_step:
            decay = self.args.ema_decay or 0.9999
            with torch.no_grad():
                for pe, p in zip(self.ema_model.parameters(), self.model.parameters()):
                    pe.lerp_(p.detach().to(pe.dtype), 1 - decay)
        return out

    def save_checkpoints(self, output_dir=None, step=None):
        path = super().save_checkpoints(output_dir, step)
        if self.rank == 0 and self.ema_model is not None:
            torch.save({k: v.cpu() for k, v in self.ema_model.state_dict().items()}, os.path.join(path, "ema.pt"))
        return path


def diff_augment(x: torch.Tensor, policy=("color", "translation", "cutout")) -> torch.Tensor:
    """Differentiable augmentation for GAN discriminators (brightness / saturation / contrast,
    random translation, random square cutout)."""
    B = x.shape[0]
    if "color" in policy:
        x = x + (torch.rand(B, 1, 1, 1, device=x.device) - 0.5)
        mean = x.mean(1, keepdim=True)
        x = (x - mean) * (torch.rand(B, 1, 1, 1, device=x.device) * 2) + mean
        mean = x.mean((1, 2, 3), keepdim=True)
        x = (x - mean) * (torch.rand(B, 1, 1, 1, device=x.device) + 0.5) + mean
    if "translation" in policy:
        r = max(int(x.shape[2] * 0.125), 1)
        dx, dy = (int(v) for v in torch.randint(-r, r + 1, (2,)))
        x = torch.roll(F.pad(x, (r, r, r, r)), shifts=(dy, dx), dims=(2, 3))[:, :, r:-r, r:-r]
    if "cutout" in policy:
        s = max(x.shape[2] // 4, 1)
        cy, cx = (int(v) for v in torch.randint(0, x.shape[2] - s + 1, (2,)))
        mask = torch.ones_like(x)
        mask[:, :, cy:cy + s, cx:cx + s] = 0
        x = x * mask
    return x


@TRAINER_REGISTER.register("rae_trainer")
class RaeTrainer(FSDP2SFTTrainer):
    """Expects a model with ``encode``, ``decode``, ``discriminator`` and ``last_layer()``."""

    def __init__(self, *a, **k):
        super().__init__(*a, **k)
        self.enable_perf_metrics = False
        cfg = dict((self.args.rl_config or {}).get("gan", {})) if self.args.rl_config else {}
        self.disc_start = int(cfg.get("disc_start", 0))
        self.disc_weight = float(cfg.get("disc_weight", 0.75))
        self.disc_steps = int(cfg.get("disc_steps", 1))
        self.perceptual_weight = float(cfg.get("perceptual_weight", 0.0))
        self.ema_state: Dict[str, torch.Tensor] = {}

    def resolve_runtime(self) -> str:
        return "torch_fsdp2" if self.world_size > 1 else "plain"

    def prepare_model(self):
        if self.world_size > 1:
            super().prepare_model()
        else:
            self.runtime_kind = "plain"
            self.model.to(self.device)

    def prepare_optimizer(self):
        a = self.args
        gen = [p for n, p in self.model.named_parameters() if p.requires_grad and "discriminator" not in n]
        disc = [p for n, p in self.model.named_parameters() if p.requires_grad and "discriminator" in n]
        kw = dict(lr=a.learning_rate, betas=(a.adam_beta1, a.adam_beta2), eps=a.adam_epsilon, weight_decay=a.weight_decay)
        self.optimizer = torch.optim.AdamW(gen, **kw)
        self.disc_optimizer = torch.optim.AdamW(disc, **kw)
        for o in (self.optimizer, self.disc_optimizer):
            for g in o.param_groups:
                g.setdefault("initial_lr", g["lr"])

    def adaptive_weight(self, rec_loss, g_loss):
        last = self.model.last_layer()
        g_rec = torch.autograd.grad(rec_loss, last, retain_graph=True)[0]
        g_gan = torch.autograd.grad(g_loss, last, retain_graph=True)[0]
        return (g_rec.norm() / (g_gan.norm() + 1e-4)).clamp(0, 1e4).detach() * self.disc_weight

    def training_step(self, batch, do_step):
        m = self.model
        m.train()
        x = batch["pixel_values"].float()
        z, hw = m.encode(x)
        rec = m.decode(z, x.shape[0], hw)
        rec_loss = (rec - x).abs().mean()
        use_gan = self.global_step >= self.disc_start
        loss = rec_loss
        if use_gan:
            g_loss = -m.discriminator(diff_augment(rec)).mean()
            loss = rec_loss + self.adaptive_weight(rec_loss, g_loss) * g_loss
        self.lr_factor = self.current_lr_factor(self.global_step)
        for o in (self.optimizer, self.disc_optimizer):
            for g in o.param_groups:
                g["lr"] = g["initial_lr"] * self.lr_factor
        self.optimizer.zero_grad(set_to_none=True)
        loss.backward()
        gn = torch.nn.utils.clip_grad_norm_([p for g in self.optimizer.param_groups for p in g["params"]], self.args.max_grad_norm)
        self.optimizer.step()
        if use_gan:
            for _ in range(self.disc_steps):
                real = m.discriminator(diff_augment(x))
                fake = m.discriminator(diff_augment(rec.detach()))
                d_loss = 0.5 * (F.relu(1 - real).mean() + F.relu(1 + fake).mean())  # hinge
                self.disc_optimizer.zero_grad(set_to_none=True)
                d_loss.backward()
                self.disc_optimizer.step()
        decay = self.args.ema_decay or 0.9999
        with torch.no_grad():
            for n, p in m.named_parameters():
                if p.requires_grad and "discriminator" not in n:
                    self.ema_state.setdefault(n, p.detach().float().clone()).lerp_(p.detach().float(), 1 - decay)
        return loss.detach(), gn

    def save_checkpoints(self, output_dir=None, step=None):
        step = self.global_step if step is None else step
        out = os.path.join(output_dir or self.args.output_dir, f"checkpoint-{step}")
        os.makedirs(out, exist_ok=True)
        if self.rank == 0:
            torch.save({k: v.cpu() for k, v in self.model.state_dict().items()}, os.path.join(out, "model.pt"))
            torch.save({k: v.cpu() for k, v in self.ema_state.items()}, os.path.join(out, "ema_state.pt"))
        return out
