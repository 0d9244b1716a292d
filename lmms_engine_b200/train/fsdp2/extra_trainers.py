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


def local_shard(t: torch.Tensor) -> torch.Tensor:
    return t.to_local() if hasattr(t, "to_local") else t


def whole_tensor(t: torch.Tensor) -> torch.Tensor:
    return t.full_tensor() if hasattr(t, "full_tensor") else t


@TRAINER_REGISTER.register("sit_trainer")
class SitTrainer(FSDP2SFTTrainer):
    def __init__(self, *a, **k):
        super().__init__(*a, **k)
        self.enable_perf_metrics = False
        self.ema_model = None

    def prepare_model(self):
        twin = copy.deepcopy(self.model)  # before a sharding wrapper is applied: a wrapped model cannot be copied
        super().prepare_model()
        self.ema_model = self.prepare_frozen_twin(twin)

    def training_step(self, batch, do_step):
        out = super().training_step(batch, do_step)
        if do_step:
            decay = self.args.ema_decay or 0.9999
            with torch.no_grad():
                for pe, p in zip(self.ema_model.parameters(), self.model.parameters()):
                    pe, p = local_shard(pe), local_shard(p)  # the twin is sharded like the model: shard meets shard
                    pe.lerp_(p.detach().to(pe.dtype), 1 - decay)
        return out

    def save_checkpoints(self, output_dir=None, step=None):
        path = super().save_checkpoints(output_dir, step)
        if self.ema_model is not None:
            full = {k: whole_tensor(v).cpu() for k, v in self.ema_model.state_dict().items()}  # a collective under sharding
            if self.rank == 0:
                torch.save(full, os.path.join(path, "ema.pt"))
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


GAN_DEFAULTS: Dict[str, Any] = {
    # the stage-1 recipe of the reference (src/lmms_engine/train/fsdp2/rae_trainer.py:28-56); schedule entries are in
    # epochs unless the ``*_step`` form is given
    "disc_weight": 0.75, "perceptual_weight": 1.0, "disc_updates": 1, "max_d_weight": 1e4, "disc_loss": "hinge",
    "gen_loss": "vanilla", "discriminator_start": 6, "discriminator_loss_start": 8, "lpips_start": 0,
    "discriminator_lr": 2e-4, "discriminator_weight_decay": 0.0, "discriminator": "dino", "dino_ckpt_path": None, "ks": 9,
    "key_depths": (2, 5, 8, 11), "norm_type": "bn", "using_spec_norm": True, "norm_eps": 1e-6, "recipe": "S_8",
    "lpips_vgg_path": None, "lpips_lin_path": None, "allow_random_critics": False, "augment": {"prob": 1.0, "cutout": 0.0},
}


@TRAINER_REGISTER.register("rae_trainer")
class RaeTrainer(FSDP2SFTTrainer):
    """Expects a model with ``encode`` / ``decode`` (or a forward returning ``out_pixels``) and ``last_layer()``.

    Generator loss = L1 + ``perceptual_weight`` x LPIPS + ``disc_weight`` x adaptive weight x adversarial term; the
    adaptive weight balances the gradient norms of the reconstruction and adversarial terms at the decoder's last
    layer.  The critics (LPIPS, DINO discriminator) live in the trainer, not in the model: the autoencoder's checkpoint
    holds the autoencoder only.  Options come from ``trainer_args.gan_config`` over ``GAN_DEFAULTS``."""

    def __init__(self, *a, **k):
        super().__init__(*a, **k)
        self.enable_perf_metrics = False
        cfg = dict(GAN_DEFAULTS)
        cfg.update(dict(getattr(self.args, "gan_config", None) or {}))
        self.gan = cfg
        self.disc_weight, self.perceptual_weight = float(cfg["disc_weight"]), float(cfg["perceptual_weight"])
        self.disc_updates, self.max_d_weight = int(cfg["disc_updates"]), float(cfg["max_d_weight"])
        self.ema_state: Dict[str, torch.Tensor] = {}
        self.discriminator = self.lpips = None
        self.loss_parts: Dict[str, float] = {}

    def resolve_runtime(self) -> str:
        return "torch_fsdp2" if self.world_size > 1 else "plain"

    # ---- set-up -------------------------------------------------------------------------------------------
    def build_critics(self):
        from ...models.rae import DinoDiscriminator, Lpips

        cfg = self.gan
        rand = bool(cfg["allow_random_critics"])
        if self.disc_weight > 0:
            if cfg["discriminator"] == "dino":
                self.discriminator = DinoDiscriminator(cfg["dino_ckpt_path"], ks=int(cfg["ks"]), key_depths=tuple(cfg["key_depths"]),
                                                       norm_type=cfg["norm_type"], using_spec_norm=bool(cfg["using_spec_norm"]),
                                                       norm_eps=float(cfg["norm_eps"]), recipe=cfg["recipe"], allow_random=rand,
                                                       backbone=cfg.get("backbone"))
            elif cfg["discriminator"] == "patch":
                from ...models.diffusion import PatchDiscriminator

                self.discriminator = PatchDiscriminator(3, int(cfg.get("disc_dim", 256)))
            else:
                raise ValueError(f"unknown discriminator '{cfg['discriminator']}' (dino | patch)")
            self.discriminator.to(self.device).train()
        if self.perceptual_weight > 0:
            self.lpips = Lpips(cfg["lpips_vgg_path"], cfg["lpips_lin_path"], allow_random=rand).to(self.device)

    def prepare_model(self):
        if self.world_size > 1:
            super().prepare_model()
        else:
            self.runtime_kind = "plain"
            self.model.to(self.device)
        self.build_critics()

    def prepare_optimizer(self):
        a = self.args
        gen = [p for p in self.model.parameters() if p.requires_grad]
        kw = dict(betas=(a.adam_beta1, a.adam_beta2), eps=a.adam_epsilon)
        self.optimizer = torch.optim.AdamW(gen, lr=a.learning_rate, weight_decay=a.weight_decay, **kw)
        opts = [self.optimizer]
        self.disc_optimizer = None
        if self.discriminator is not None:
            disc = [p for p in self.discriminator.parameters() if p.requires_grad]
            self.disc_optimizer = torch.optim.AdamW(disc, lr=float(self.gan["discriminator_lr"]),
                                                    weight_decay=float(self.gan["discriminator_weight_decay"]), **kw)
            opts.append(self.disc_optimizer)
        for o in opts:
            for g in o.param_groups:
                g.setdefault("initial_lr", g["lr"])

    def _start_step(self, name: str) -> int:
        if f"{name}_step" in self.gan:
            return int(self.gan[f"{name}_step"])
        return int(float(self.gan[name]) * (self.steps_per_epoch() or 0))

    # ---- losses -------------------------------------------------------------------------------------------
    def augment(self, x):
        aug = self.gan.get("augment") or {}
        if float(aug.get("prob", 1.0)) <= 0 or torch.rand(()) > float(aug.get("prob", 1.0)):
            return x
        policy = ("color", "translation") + (("cutout",) if float(aug.get("cutout", 0.0)) > 0 else ())
        return diff_augment(x, policy)

    def adaptive_weight(self, rec_loss, g_loss):
        """Ratio of the two terms' gradient norms at the last layer's weight.  The gradient is formed from the layer's
        recorded input and output (``d_output^T @ input``): under a sharding wrapper the weight that took part in the
        pass is a gathered temporary, so differentiating with respect to the module's (sharded) parameter finds nothing
        (the reference differentiates the parameter with ``allow_unused``, src/lmms_engine/train/fsdp2/rae_trainer.py:446-472)."""
        io = self.model.last_layer_io() if hasattr(self.model, "last_layer_io") else None
        if io is None:
            last = self.model.last_layer()
            g_rec = torch.autograd.grad(rec_loss, last, retain_graph=True)[0]
            g_gan = torch.autograd.grad(g_loss, last, retain_graph=True)[0]
        else:
            x, y = io
            rows = x.detach().reshape(-1, x.shape[-1]).float()
            g_rec, g_gan = (torch.autograd.grad(loss, y, retain_graph=True)[0].reshape(-1, y.shape[-1]).float().t() @ rows
                            for loss in (rec_loss, g_loss))
        return (g_rec.norm() / (g_gan.norm() + 1e-6)).clamp(0, self.max_d_weight).detach()

    def gen_loss(self, logits_fake):
        if self.gan["gen_loss"] == "hinge":
            return -logits_fake.mean()
        return F.softplus(-logits_fake).mean()  # "vanilla": non-saturating

    def disc_loss(self, real, fake):
        if self.gan["disc_loss"] == "hinge":
            return 0.5 * (F.relu(1 - real).mean() + F.relu(1 + fake).mean())
        return 0.5 * (F.softplus(-real).mean() + F.softplus(fake).mean())

    def reconstruct(self, x):
        m = self.model
        out = m(pixel_values=x)
        return out["out_pixels"] if "out_pixels" in out else out["reconstruction"]

    def training_step(self, batch, do_step):
        m = self.model
        m.train()
        x = batch["pixel_values"].float()
        rec = self.reconstruct(x).float()
        rec_loss = (rec - x).abs().mean()
        lp = rec_loss.new_zeros(())
        if self.lpips is not None and self.global_step >= self._start_step("lpips_start"):
            lp = self.lpips(rec * 2 - 1, x * 2 - 1)
        loss = rec_loss + self.perceptual_weight * lp
        g_loss = aw = rec_loss.new_zeros(())
        if self.discriminator is not None and self.global_step >= self._start_step("discriminator_loss_start"):
            self.discriminator.eval()
            g_loss = self.gen_loss(self.discriminator(self.augment(rec * 2 - 1)))
            aw = self.adaptive_weight(loss, g_loss)
            loss = loss + self.disc_weight * aw * g_loss
        self.lr_factor = self.current_lr_factor(self.global_step)
        for o in (self.optimizer, self.disc_optimizer):
            for g in (o.param_groups if o is not None else ()):
                g["lr"] = g["initial_lr"] * self.lr_factor
        self.optimizer.zero_grad(set_to_none=True)
        loss.backward()
        gn = torch.nn.utils.clip_grad_norm_([p for g in self.optimizer.param_groups for p in g["params"]], self.args.max_grad_norm)
        self.optimizer.step()
        d_total = 0.0
        if self.discriminator is not None and self.global_step >= self._start_step("discriminator_start"):
            self.discriminator.train()
            fake = (rec.detach() * 2 - 1).clamp(-1, 1)
            fake = torch.round((fake + 1) * 127.5) / 127.5 - 1  # what an 8-bit image of the reconstruction would hold
            for _ in range(max(self.disc_updates, 1)):
                d_loss = self.disc_loss(self.discriminator(self.augment(x * 2 - 1)), self.discriminator(self.augment(fake)))
                self.disc_optimizer.zero_grad(set_to_none=True)
                d_loss.backward()
                if self.world_size > 1:  # the critic is replicated: average its gradients
                    for p in self.discriminator.parameters():
                        if p.grad is not None:
                            dist.all_reduce(p.grad, op=dist.ReduceOp.AVG)
                self.disc_optimizer.step()
                d_total += float(d_loss.detach())
        self.loss_parts = {"l1_loss": float(rec_loss.detach()), "lpips_loss": float(lp.detach()), "gan_loss": float(g_loss.detach()),
                           "adaptive_weight": float(aw), "disc_loss": d_total / max(self.disc_updates, 1)}
        decay = self.args.ema_decay or 0.9978
        with torch.no_grad():
            for n, p in m.named_parameters():
                if p.requires_grad:
                    q = local_shard(p.detach()).float()  # every rank averages the shard it holds
                    self.ema_state.setdefault(n, q.clone()).lerp_(q, 1 - decay)
        return loss.detach(), gn

    @staticmethod
    def _whole_like(param, shard):
        """The whole tensor of which ``shard`` is this rank's part, laid out like ``param``."""
        if not hasattr(param, "to_local"):
            return shard
        from torch.distributed.tensor import DTensor

        return DTensor.from_local(shard, param.device_mesh, param.placements, run_check=False).full_tensor()

    def calculate_training_metrics(self, seqlens, step_seconds):
        out = super().calculate_training_metrics(seqlens, step_seconds)
        out.update({f"train/{k}": v for k, v in self.loss_parts.items()})
        return out

    def save_checkpoints(self, output_dir=None, step=None):
        step = self.global_step if step is None else step
        out = os.path.join(output_dir or self.args.output_dir, f"checkpoint-{step}")
        os.makedirs(out, exist_ok=True)
        weights = {k: whole_tensor(v).cpu() for k, v in self.model.state_dict().items()}  # collectives under sharding: every rank
        params = dict(self.model.named_parameters())
        ema = {k: self._whole_like(params[k], v).cpu() for k, v in self.ema_state.items()}
        if self.rank == 0:
            torch.save(weights, os.path.join(out, "model.pt"))
            torch.save(ema, os.path.join(out, "ema_state.pt"))
            if self.discriminator is not None:
                heads = {k: v.cpu() for k, v in self.discriminator.state_dict().items() if not k.startswith("dino.")}
                torch.save({"discriminator": heads, "optimizer": self.disc_optimizer.state_dict()}, os.path.join(out, "discriminator.pt"))
        return out
