"""``fsdp2_trainer``: the engine's own sharded-data-parallel SFT loop.

Public surface and behaviour follow the reference trainer
(src/lmms_engine/train/fsdp2/fsdp2_trainer.py:48-735): constructor
``(model, args, data_collator, train_dataset, eval_dataset, processing_class)``,
overridable ``prepare_model / prepare_dataloader / prepare_optimizer / prepare_scheduler /
compute_loss / training_step / save_checkpoints / load_checkpoints``, schedulers
``cosine | wsd | constant``, gradient accumulation, non-finite-gradient step skipping, EMA,
per-step metrics (loss, lr, grad_norm, MFU, tokens/s, sequence-length stats), the
checkpoint directory layout with rotation and auto-resume, profilers, async eval hook.

What is different by design:

* three sharding runtimes: ``native`` (replicated bf16 weights + owner-sharded optimizer,
  ``parallel/owner_sharded.py``), ``native_sharded`` (parameters sharded by owner as well and
  gathered block by block over peer memory, ``parallel/param_sharded.py``) and ``torch_fsdp2``
  (stock ``fully_shard``);
* AdamW **and Muon** are available here (the reference wires Muon only into its HF trainer);
* the step makes no host round trip: loss, grad-norm, clip coefficient and the skip flag
  stay on the device and are read back only when a step is logged; step time is measured
  with CUDA events (the reference uses ``perf_counter`` and five ``.item()`` syncs per step).
"""
from __future__ import annotations

import json
import math
import os
import random
import time
from typing import Any, Dict, List, Optional

import numpy as np
import torch
import torch.distributed as dist
from torch.utils.data import DataLoader, DistributedSampler, IterableDataset

from ...models.utils import FlopsCounter
from ...ops import muon as muon_ops
from ...parallel import process_group_manager as pgm_mod
from ...parallel.owner_sharded import OwnerShardedRuntime
from ...utils import schedulers
from ...utils.compute_tracker import ComputeTracker
from ...utils.ema_utils import EMAHelper
from ...utils import failure
from ...utils.logging_utils import logger
from ...utils.profiler import CudaEventProfiler, MemorySnapshotProfiler, StepProfiler
from ...utils.tracking import Tracking
from ...utils.train_utils import TrainUtilities, send_to_device, str_to_dtype
from .. import checkpoint as ckpt
from ..registry import TRAINER_REGISTER


def _dist_ready() -> bool:
    return dist.is_available() and dist.is_initialized()


@TRAINER_REGISTER.register("fsdp2_trainer")
class FSDP2SFTTrainer:
    def __init__(self, model, args, data_collator=None, train_dataset=None, eval_dataset=None, processing_class=None):
        self.model = model
        self.args = args
        self.data_collator = data_collator
        self.train_dataset = train_dataset
        self.eval_dataset = eval_dataset
        self.processing_class = processing_class
        self.pgm = pgm_mod.process_group_manager
        self.rank = dist.get_rank() if _dist_ready() else 0
        self.world_size = dist.get_world_size() if _dist_ready() else 1
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        use_cuda = torch.cuda.is_available() and not args.use_cpu
        self.device = torch.device("cuda", self.local_rank) if use_cuda else torch.device("cpu")
        if use_cuda:
            torch.cuda.set_device(self.device)
        self.global_step = 0
        self.total_tokens = 0
        self.accumulated_grad_steps = 0
        self.runtime: Optional[OwnerShardedRuntime] = None
        self.optimizer = None
        self.lr_factor = 1.0
        self.ema: Optional[EMAHelper] = None
        self.eval_backend = None
        self.should_stop = False
        self.flops_counter = FlopsCounter(getattr(model, "config", {}))
        self.compute_tracker = ComputeTracker(self.world_size, args.carbon_intensity or 0.475)
        self.tracking: Optional[Tracking] = None
        self.log_history: List[Dict[str, Any]] = []
        self.enable_perf_metrics = True
        self._acc_tokens, self._acc_flops, self._acc_t0 = 0.0, 0.0, time.perf_counter()

    # ------------------------------------------------------------------ helpers
    @property
    def dp_rank(self) -> int:
        return self.pgm.dp_rank if self.pgm is not None else 0

    @property
    def dp_size(self) -> int:
        return self.pgm.dp_size if self.pgm is not None else 1

    @property
    def sp_size(self) -> int:
        return self.pgm.cp_size if self.pgm is not None else 1

    @property
    def is_native(self) -> bool:
        return getattr(self, "runtime_kind", None) in ("native", "native_sharded")

    def compute_dtype(self) -> torch.dtype:
        if self.args.bf16:
            return torch.bfloat16
        if self.args.fp16:
            return torch.float16
        return torch.float32

    def resolve_runtime(self) -> str:
        rt = self.args.sharding_runtime or "auto"
        if rt != "auto":
            return rt
        if self.pgm is not None and (self.pgm.enable_tp or self.pgm.enable_ep or self.pgm.enable_hsdp):
            return "torch_fsdp2"
        if self.device.type == "cpu" and self.world_size > 1:
            return "torch_fsdp2"
        return "native"

    # ------------------------------------------------------------------ model / optimizer
    def prepare_model(self):
        args = self.args
        dtype = self.compute_dtype()
        self.runtime_kind = self.resolve_runtime()
        if args.gradient_checkpointing and hasattr(self.model, "gradient_checkpointing_enable"):
            self.model.gradient_checkpointing_enable()
        if self.sp_size > 1 and self.pgm is not None:
            self.model.sp_group = self.pgm.cp_group
        if getattr(self.model, "vit_frame_parallel", False) and self.pgm is not None and self.world_size > 1:
            self.model.vit_group = self.pgm.dp_cp_group
        if self.is_native:
            self.model.to(device=self.device, dtype=dtype)
            return
        # ---- stock FSDP2 (ZeRO-3), also the path for TP / EP / HSDP meshes ------------------
        from torch.distributed.fsdp import fully_shard

        from ...parallel.parallelize import apply_parallelize, has_parallel_plan

        model_type = getattr(getattr(self.model, "config", None), "model_type", None)
        if self.pgm is not None and self.pgm.enable_parallel and has_parallel_plan(model_type):
            if self.pgm.enable_hsdp:
                raise ValueError("HSDP cannot be combined with TP / EP")
            self.model.to(self.device)
            apply_parallelize(self.model, model_type, args, dtype)
            return
        self.model.to(self.device)
        from ...parallel.plans import mixed_precision_policy

        mp = mixed_precision_policy(args, dtype)
        mesh = self.pgm.fsdp_mesh
        fsdp_cfg = args.fsdp_config or {}
        kw = dict(mesh=mesh, reshard_after_forward=bool(fsdp_cfg.get("reshard_after_forward", True)))
        if mp is not None:
            kw["mp_policy"] = mp
        wrap_names = set(fsdp_cfg.get("transformer_layer_cls_to_wrap") or getattr(self.model, "_no_split_modules", []) or [])
        for module in self.model.modules():
            if type(module).__name__ in wrap_names:
                fully_shard(module, **kw)
        root_mp = mixed_precision_policy(args, dtype, root=True)
        if root_mp is not None:
            kw["mp_policy"] = root_mp
        fully_shard(self.model, **kw)

    def prepare_frozen_twin(self, twin):
        """Give ``twin`` (a copy of the model taken BEFORE ``prepare_model``) the model's placement - device, dtype, and
        under torch FSDP2 the same sharding wrappers - and freeze it: EMA weights, the reference policy of GRPO."""
        keep = self.model
        self.model = twin
        try:
            FSDP2SFTTrainer.prepare_model(self)
        finally:
            self.model = keep
        return twin.requires_grad_(False).eval()

    def native_grad_dtype(self) -> torch.dtype:
        """Dtype of the native runtime's flat gradient buffer (accumulation across micro-batches and the
        cross-rank sum): ``reduce_dtype`` when it asks for fp32, the compute dtype otherwise."""
        want = str_to_dtype(self.args.reduce_dtype) if self.args.reduce_dtype else None
        return torch.float32 if want == torch.float32 else self.compute_dtype()

    def build_param_groups(self):
        """AdamW groups, or the four Muon/Adam x decay/no-decay groups when ``use_muon``."""
        decay, no_decay, mu = [], [], []
        for name, p in self.model.named_parameters():
            if not p.requires_grad:
                continue
            if self.args.use_muon and muon_ops.is_muon_param(name, p):
                mu.append(p)
            elif p.ndim >= 2 and "bias" not in name and "norm" not in name:
                decay.append(p)
            else:
                no_decay.append(p)
        return decay, no_decay, mu

    def prepare_optimizer(self):
        args = self.args
        if self.is_native:
            group = self.pgm.dp_cp_group if (self.pgm is not None and self.world_size > 1) else None
            comm = None
            if self.device.type == "cuda" and self.world_size > 1 and os.environ.get("LMMS_B200_PEER_COMM", "1") != "0":
                from ...parallel.peer_comm import PeerComm

                # a device-side wait for a peer gives up after the job's collective timeout, like NCCL would
                timeout_ms = int(max(float(args.ddp_timeout or 1800), 1.0) * 1000)
                try:
                    comm = PeerComm(group, self.device, barrier_timeout_ms=timeout_ms)
                except Exception as e:
                    # ranks on different hosts (no peer mapping) are a configuration the operator must choose
                    # on purpose: the NCCL path is a different, slower runtime
                    if os.environ.get("LMMS_B200_PEER_COMM", "1") != "auto":
                        raise RuntimeError(
                            "peer-memory communication could not be set up for the native runtime "
                            f"({type(e).__name__}: {e}); set LMMS_B200_PEER_COMM=0 to run it on torch.distributed "
                            "collectives, or LMMS_B200_PEER_COMM=auto to fall back with a warning") from e
                    logger.warning(f"peer-memory communication unavailable ({e}); using torch.distributed collectives")
            runtime_cls = OwnerShardedRuntime
            if self.runtime_kind == "native_sharded":
                from ...parallel.param_sharded import ParamShardedRuntime as runtime_cls
            self.runtime = runtime_cls(
                self.model, group, lr=args.learning_rate, weight_decay=args.weight_decay,
                betas=(args.adam_beta1, args.adam_beta2), eps=args.adam_epsilon, max_grad_norm=args.max_grad_norm,
                use_muon=bool(args.use_muon), muon_momentum=args.muon_momentum, muon_nesterov=args.muon_nesterov,
                muon_ns_steps=args.muon_ns_steps, param_dtype=self.compute_dtype(), device=self.device, comm=comm,
                grad_dtype=self.native_grad_dtype(),
            )
            return
        decay, no_decay, mu = self.build_param_groups()
        if args.use_muon:
            from ...utils.muon_utils import Muon

            groups = [
                dict(params=mu, use_muon=True, lr=args.learning_rate, weight_decay=args.weight_decay,
                     momentum=args.muon_momentum, nesterov=args.muon_nesterov, ns_steps=args.muon_ns_steps),
                dict(params=decay, use_muon=False, lr=args.learning_rate, weight_decay=args.weight_decay,
                     betas=(args.adam_beta1, args.adam_beta2), eps=args.adam_epsilon),
                dict(params=no_decay, use_muon=False, lr=args.learning_rate, weight_decay=0.0,
                     betas=(args.adam_beta1, args.adam_beta2), eps=args.adam_epsilon),
            ]
            self.optimizer = Muon([g for g in groups if g["params"]])
        else:
            # one group per (weight decay, device mesh): the fused kernel of a group then sees tensors of one kind
            # (expert parameters live on another mesh than the rest).  Fused: one pass over parameters and moments
            # instead of the seven of the per-operation ("foreach") implementation - a fifth of the step of the
            # expert-parallel configuration was spent there.
            def by_mesh(params, wd):
                groups: Dict[Any, list] = {}
                for p_ in params:
                    groups.setdefault(id(getattr(p_, "device_mesh", None)), []).append(p_)
                return [dict(params=ps, weight_decay=wd) for ps in groups.values()]

            every = decay + no_decay
            fused = bool(every) and all(p_.is_cuda for p_ in every) and os.environ.get("LMMS_B200_FUSED_ADAMW", "1") != "0"
            self.optimizer = torch.optim.AdamW(
                by_mesh(decay, args.weight_decay) + by_mesh(no_decay, 0.0),
                lr=args.learning_rate, betas=(args.adam_beta1, args.adam_beta2), eps=args.adam_epsilon, fused=fused,
            )
        for g in self.optimizer.param_groups:
            g.setdefault("initial_lr", g["lr"])

    def prepare_scheduler(self, total_steps: int):
        args = self.args
        self.total_steps = total_steps
        self.warmup_steps = int(args.warmup_ratio * total_steps) if args.warmup_ratio > 0 else int(args.warmup_steps)
        self.sched_kwargs = dict(args.lr_scheduler_kwargs or {})

    def current_lr_factor(self, step: int) -> float:
        return schedulers.lr_factor(self.args.lr_scheduler_type, step, self.warmup_steps, self.total_steps, **self.sched_kwargs)

    # ------------------------------------------------------------------ data
    def prepare_dataloader(self):
        args = self.args
        ds = self.train_dataset
        kw: Dict[str, Any] = dict(batch_size=args.per_device_train_batch_size, collate_fn=self.data_collator,
                                  num_workers=args.dataloader_num_workers, drop_last=args.dataloader_drop_last,
                                  pin_memory=bool(args.dataloader_pin_memory) and self.device.type == "cuda")
        if args.dataloader_num_workers > 0 and args.dataloader_prefetch_factor:
            kw["prefetch_factor"] = args.dataloader_prefetch_factor
        self.sampler = None
        if not isinstance(ds, IterableDataset):
            # samplers work on DATA-parallel ranks: the ranks of a sequence-/tensor-parallel group read the same samples
            lengths = None
            if args.group_by_length:
                from ..samplers import LengthGroupedSampler, dataset_lengths

                lengths = dataset_lengths(ds)
                if lengths is None:
                    logger.warning("group_by_length is set but the dataset exposes no modality_length / lengths; sampling uniformly")
            if lengths is not None:
                self.sampler = LengthGroupedSampler(lengths, args.per_device_train_batch_size, num_replicas=self.dp_size,
                                                    rank=self.dp_rank, seed=args.seed, drop_last=args.dataloader_drop_last)
            else:
                self.sampler = DistributedSampler(ds, num_replicas=self.dp_size, rank=self.dp_rank, shuffle=True,
                                                  seed=args.seed, drop_last=args.dataloader_drop_last)
            kw["sampler"] = self.sampler
        try:
            from torchdata.stateful_dataloader import StatefulDataLoader

            self.dataloader = StatefulDataLoader(ds, **kw)
        except Exception:
            self.dataloader = DataLoader(ds, **kw)
        return self.dataloader

    def steps_per_epoch(self) -> Optional[int]:
        try:
            return max(len(self.dataloader) // max(self.args.gradient_accumulation_steps, 1), 1)
        except TypeError:
            return None

    # ------------------------------------------------------------------ step
    def compute_loss(self, batch: Dict[str, Any]) -> torch.Tensor:
        if self.device.type == "cuda" and not self.is_native and self.compute_dtype() != torch.float32:
            with torch.autocast("cuda", dtype=self.compute_dtype()):
                out = self.model(**batch)
        else:
            out = self.model(**batch)
        loss = out["loss"] if isinstance(out, dict) else out[0]
        self._last_out = out
        return loss

    def training_step(self, batch: Dict[str, Any], do_step: bool):
        """One micro-batch forward/backward; on ``do_step`` also clip, update and schedule.
        Returns device scalars ``(loss, grad_norm or None)``."""
        args = self.args
        self.model.train()
        rt = self.runtime
        if rt is not None and getattr(rt, "breakdown", False):
            rt.phase_events = []
            rt._mark("start")
        loss = self.compute_loss(batch)
        if rt is not None and getattr(rt, "breakdown", False):
            rt._mark("forward")
        if do_step and self.runtime is not None:
            self.runtime.arm()  # this backward finishes the step's gradients: reduce them bucket by bucket as they complete
        (loss / args.gradient_accumulation_steps).backward()
        if self.runtime is not None:
            self.runtime.after_backward()
        self.accumulated_grad_steps += 1
        grad_norm = None
        if do_step:
            self.lr_factor = self.current_lr_factor(self.global_step)
            if self.runtime is not None:
                grad_norm = self.runtime.step(self.lr_factor)
            else:
                from ...utils.fsdp2_utils import fsdp2_clip_grad_norm_

                if self.pgm is not None and self.pgm.enable_tp:
                    from ...parallel import tp_ops

                    tp_ops.sync_replicated_grads(self.model, self.pgm.tp_group)
                grad_norm = fsdp2_clip_grad_norm_(self.model.parameters(), args.max_grad_norm)
                for g in self.optimizer.param_groups:
                    g["lr"] = g["initial_lr"] * self.lr_factor
                if torch.isfinite(grad_norm).all():
                    self.optimizer.step()
                else:
                    logger.warning(f"step {self.global_step}: non-finite grad norm, skipping optimizer step")
                self.optimizer.zero_grad(set_to_none=True)
            self.accumulated_grad_steps = 0
            if self.ema is not None:
                self.ema.update(self.global_step + 1)
        return loss.detach(), grad_norm

    # ------------------------------------------------------------------ metrics
    def batch_seqlens(self, batch) -> List[int]:
        if "cu_seqlens" in batch:
            cu = batch["cu_seqlens"]
            return (cu[1:] - cu[:-1]).tolist()
        if "attention_mask" in batch:
            return batch["attention_mask"].sum(-1).tolist()
        if "input_ids" in batch:
            return [int(batch["input_ids"].numel())]
        first = next((v for v in batch.values() if torch.is_tensor(v)), None)
        return [int(first.shape[0])] if first is not None else [0]

    def calculate_training_metrics(self, seqlens: List[int], step_seconds: float) -> Dict[str, Any]:
        ntok = float(sum(seqlens))
        flops = self.flops_counter.flops_per_step(seqlens)
        promised = TrainUtilities.get_device_flops("B")
        sp_tp = self.sp_size * (self.pgm.tp_size if self.pgm is not None else 1)
        mfu = flops / max(step_seconds, 1e-9) / sp_tp / promised if math.isfinite(promised) else 0.0
        # tokens and FLOPs of the steps since the last logged one were counted on the host, step by step
        # (count_step); only the exchange between ranks waits for a logged step
        acc_tok, acc_flops, acc_s = self._acc_tokens, self._acc_flops, max(time.perf_counter() - self._acc_t0, step_seconds)
        self._acc_tokens, self._acc_flops, self._acc_t0 = 0.0, 0.0, time.perf_counter()
        stats = torch.tensor([mfu, ntok, flops, acc_tok, acc_flops], dtype=torch.float64, device=self.device)
        if self.world_size > 1:
            gathered = torch.empty(self.world_size * 5, dtype=torch.float64, device=self.device)
            dist.all_gather_into_tensor(gathered, stats)
            g = gathered.view(self.world_size, 5)
        else:
            g = stats.view(1, 5)
        toks = g[:, 1] / self.sp_size
        total = float(toks.sum())
        window_tokens = float(g[:, 3].sum()) / self.sp_size
        self.total_tokens += int(window_tokens)
        self.compute_tracker.update(float(g[:, 4].sum()) / sp_tp, int(window_tokens), acc_s)
        return {
            "train/mfu": float(g[:, 0].mean()),
            "perf/global_seq_len_avg": float(g[:, 1].mean()),
            "perf/global_seq_len_min": float(g[:, 1].min()),
            "perf/global_seq_len_max": float(g[:, 1].max()),
            "train/total_tokens": self.total_tokens,
            "train/tokens_per_second": total / max(step_seconds, 1e-9),
            "train/tokens_per_gpu": total / max(step_seconds, 1e-9) / self.world_size,
        }

    def count_step(self, seqlens: List[int]) -> None:
        """Host-side token and FLOP counters, updated on EVERY optimizer step from lengths the host already
        knows (no device sync), so that ``logging_steps > 1`` does not undercount what is persisted."""
        self._acc_tokens += float(sum(seqlens))
        self._acc_flops += float(self.flops_counter.flops_per_step(seqlens))

    def extra_metrics(self) -> Dict[str, Any]:
        """Trainer-specific values merged into every logged step."""
        return {}

    def check_device_status(self, heartbeat=None) -> None:
        """Read the status word that bounded device-side waits raise (a peer barrier that ran out, a
        fused collective that gave up).  The step in which it was raised applied no update (the word
        feeds the optimizer's skip flag), so the weights are intact; training must not go on."""
        if self.device.type != "cuda":
            return
        from ...ops import _cuda

        try:
            _cuda.check_status(self.device)
        except RuntimeError as e:
            if heartbeat is not None:
                heartbeat.report_error(self.global_step, f"device status: {e}")
            raise

    # ------------------------------------------------------------------ checkpoints
    def _full_model_state(self) -> Dict[str, torch.Tensor]:
        return {k: v for k, v in self.model.state_dict().items()}

    def _iter_full_model_state(self):
        """``(state-dict key, full tensor)`` pairs; tensors of a parameter-sharded runtime are valid only
        until the next pair is requested."""
        if hasattr(self.runtime, "full_state_items"):
            by_param = {id(p): k for k, p in self.model.state_dict(keep_vars=True).items()}
            aliases: Dict[str, List[str]] = {}
            for k, p in self.model.state_dict(keep_vars=True).items():
                aliases.setdefault(by_param[id(p)], []).append(k)
            params = dict(self.model.named_parameters())
            seen = set()
            for name, full in self.runtime.full_state_items():
                canon = by_param.get(id(params[name]), name)
                for k in aliases.get(canon, [name]):  # tied weights appear under every one of their keys
                    seen.add(k)
                    yield k, full
            for k, v in self.model.state_dict().items():  # persistent buffers
                if k not in seen:
                    yield k, v
            return
        yield from self._full_model_state().items()

    def save_checkpoints(self, output_dir: Optional[str] = None, step: Optional[int] = None) -> str:
        args = self.args
        step = self.global_step if step is None else step
        out = os.path.join(output_dir or args.output_dir, f"checkpoint-{step}")
        os.makedirs(out, exist_ok=True)
        W, r = self.world_size, self.rank
        ckpt.barrier()
        if self.is_native:
            mesh = self.pgm.device_mesh["fsdp"] if self.pgm is not None else None
            model_sd = {}
            # one tensor at a time: a sharded runtime materialises a block's parameters only while they are consumed
            for name, full in self._iter_full_model_state():
                if mesh is not None:
                    model_sd.update(ckpt.shard0_dtensor_state({name: full}, mesh))
                else:
                    model_sd[name] = full.detach().cpu().clone()
            opt_sd = self.runtime.state_dict()
        else:
            model_sd = self.model.state_dict()
            opt_sd = self.optimizer.state_dict()
        ckpt.save_rank_state(out, ckpt.MODEL_DIR, "model", W, r, model_sd)
        if self.ema is not None and self.ema.initialized:
            ckpt.save_rank_state(out, ckpt.EMA_DIR, "model", W, r, self.ema.state_dict())
        if not args.save_only_model:
            ckpt.save_rank_state(out, "optimizer", "optimizer", W, r, opt_sd)
            extra = {
                "lr_scheduler_state": {"global_step": self.global_step, "lr_factor": self.lr_factor},
                "rng": {"cpu": torch.get_rng_state(), "numpy": np.random.get_state(), "random": random.getstate(),
                        "cuda": torch.cuda.get_rng_state() if self.device.type == "cuda" else None},
                "total_tokens": self.total_tokens,
                "accumulated_grad_steps": self.accumulated_grad_steps,
                "compute_tracker": self.compute_tracker.state_dict(),
                "global_step": self.global_step,
            }
            ckpt.save_rank_state(out, "extra_state", "extra_state", W, r, extra)
            dl_state = None
            if hasattr(self.dataloader, "state_dict"):
                try:
                    dl_state = self.dataloader.state_dict()
                except Exception:
                    dl_state = None
            if dl_state is None and hasattr(self.train_dataset, "state_dict"):
                dl_state = {"dataset_state": self.train_dataset.state_dict()}
            ckpt.save_rank_state(out, "dataloader_state", "dataloader_state", W, r, dl_state)
        if r == 0:
            cfg = getattr(self.model, "config", None)
            if cfg is not None:
                with open(os.path.join(out, "config.json"), "w") as f:
                    json.dump(cfg.to_dict() if hasattr(cfg, "to_dict") else dict(cfg), f, indent=2, default=str)
            if self.processing_class is not None and hasattr(self.processing_class, "save_pretrained"):
                try:
                    self.processing_class.save_pretrained(out)
                except Exception as e:
                    logger.warning(f"could not save processor: {e}")
        ckpt.barrier()  # every rank's files are on disk
        if r == 0:
            # the marker makes the checkpoint eligible for resume; a job that dies before this line leaves
            # a directory that resume skips
            failure.write_completion_marker(out)
            ckpt.rotate_checkpoints(output_dir or args.output_dir, args.save_total_limit)
        ckpt.barrier()
        return out

    def load_checkpoints(self, path: str) -> None:
        W, r = self.world_size, self.rank
        saved_w = ckpt.saved_world_size(path)
        if self.is_native:
            full = ckpt.load_full_model_state(path)
            if hasattr(self.runtime, "load_full_state"):
                self.runtime.load_full_state(full)
            else:
                own = self.model.state_dict()
                with torch.no_grad():
                    for k, v in full.items():
                        if k in own:
                            own[k].copy_(v.to(own[k].dtype))
            self.runtime.refresh_master_from_params()
            if saved_w == W and os.path.exists(os.path.join(path, "optimizer", ckpt.rank_file("optimizer", W, r))):
                self.runtime.load_state_dict(ckpt.load_rank_state(path, "optimizer", "optimizer", W, r))
            elif not self.args.save_only_model:
                logger.warning(f"optimizer state of {path} was written by {saved_w} ranks and is not loaded into this "
                               f"run of {W} ranks: AdamW moments and Muon momentum start from zero")
        else:
            if saved_w != W:
                raise ValueError(f"torch_fsdp2 checkpoints resume only at the saved world size ({saved_w})")
            self.model.load_state_dict(ckpt.load_rank_state(path, ckpt.MODEL_DIR, "model", W, r))
            opt_file = os.path.join(path, "optimizer", ckpt.rank_file("optimizer", W, r))
            if os.path.exists(opt_file):
                self.optimizer.load_state_dict(ckpt.load_rank_state(path, "optimizer", "optimizer", W, r))
        if self.ema is not None and os.path.isdir(os.path.join(path, ckpt.EMA_DIR)) and saved_w == W:
            self.ema.load_state_dict(ckpt.load_rank_state(path, ckpt.EMA_DIR, "model", W, r))
            if self.args.ema_resume_from_ema:
                self.ema.copy_to_model()
        extra_file = os.path.join(path, "extra_state", ckpt.rank_file("extra_state", saved_w, min(r, saved_w - 1)))
        if os.path.exists(extra_file):
            extra = torch.load(extra_file, map_location="cpu", weights_only=False)
            self.global_step = int(extra.get("global_step", extra["lr_scheduler_state"].get("global_step", 0)))
            self.total_tokens = int(extra.get("total_tokens", 0))
            self.accumulated_grad_steps = int(extra.get("accumulated_grad_steps", 0))
            self.compute_tracker.load_state_dict(extra.get("compute_tracker", {}))
            if saved_w == W:
                rng = extra.get("rng", {})
                if rng.get("cpu") is not None:
                    torch.set_rng_state(rng["cpu"])
                if rng.get("numpy") is not None:
                    np.random.set_state(rng["numpy"])
                if rng.get("random") is not None:
                    random.setstate(rng["random"])
                if rng.get("cuda") is not None and self.device.type == "cuda":
                    torch.cuda.set_rng_state(rng["cuda"])
        dl_file = os.path.join(path, "dataloader_state", ckpt.rank_file("dataloader_state", W, r))
        if saved_w == W and os.path.exists(dl_file):
            st = torch.load(dl_file, map_location="cpu", weights_only=False)
            if st is not None:
                if "dataset_state" in st and hasattr(self.train_dataset, "load_state_dict") and len(st) == 1:
                    self.train_dataset.load_state_dict(st["dataset_state"])
                elif hasattr(self.dataloader, "load_state_dict"):
                    self.dataloader.load_state_dict(st)
        logger.info(f"resumed from {path} at step {self.global_step}")

    # ------------------------------------------------------------------ eval hook
    def validation_step(self, checkpoint_path: str) -> None:
        if self.eval_backend is not None and self.rank == 0:
            self.eval_backend.submit(checkpoint_path, self.global_step)

    def _check_eval_results(self) -> None:
        if self.eval_backend is None or self.rank != 0:
            return
        for step, metrics in self.eval_backend.poll_results():
            if self.tracking is not None:
                self.tracking.log({**metrics, "global_step": step}, step=self.global_step)

    # ------------------------------------------------------------------ main loop
    def train(self, resume_from_checkpoint: Optional[str] = None):
        args = self.args
        self.prepare_model()
        self.prepare_dataloader()
        self.prepare_optimizer()
        spe = self.steps_per_epoch()
        if args.max_steps and args.max_steps > 0:
            total_steps = args.max_steps
        elif spe is not None:
            total_steps = int(math.ceil(args.num_train_epochs * spe))
        else:
            raise ValueError("iterable datasets need max_steps > 0")
        self.prepare_scheduler(total_steps)
        if args.ema_enabled:
            self.ema = EMAHelper(self.model, args.ema_decay, args.ema_update_every, args.ema_start_step,
                                 args.ema_requires_grad_only, args.ema_param_filter)
        if args.eval_config:
            from ...eval.backends import EvalServerBackend

            self.eval_backend = EvalServerBackend(args.eval_config, args.output_dir) if self.rank == 0 else None
        if resume_from_checkpoint:
            self.load_checkpoints(resume_from_checkpoint)
        if self.ema is not None:
            self.ema.maybe_init()
        if self.rank == 0:
            report = args.report_to if isinstance(args.report_to, (list, tuple)) else [args.report_to]
            self.tracking = Tracking(os.environ.get("WANDB_PROJECT"), args.run_name, [b for b in report if b] + ["console"],
                                     config=args.to_dict(), output_dir=args.output_dir)
        prof = StepProfiler(args.enable_profiler, args.output_dir, args.profiler_config, self.rank)
        mem_prof = MemorySnapshotProfiler(args.enable_memory_snapshot, args.output_dir, args.memory_snapshot_config, self.rank)
        ev_prof = CudaEventProfiler(args.enable_cuda_event_profiler, args.output_dir, args.cuda_event_profiler_config, self.rank)
        prof.start()
        mem_prof.start()
        ga = max(args.gradient_accumulation_steps, 1)
        cuda = self.device.type == "cuda"
        heartbeat = None
        if getattr(args, "heartbeat_timeout", 0) and self.world_size > 1 and dist.is_initialized():
            store = dist.distributed_c10d._get_default_store()
            heartbeat = failure.Heartbeat(store, self.rank, self.world_size, float(args.heartbeat_timeout))
        epoch = 0
        micro = 0
        seqlens_acc: List[int] = []
        t_host = time.perf_counter()
        ev0 = ev1 = None
        loss_acc = None
        while not self.should_stop:
            if self.sampler is not None:
                self.sampler.set_epoch(epoch)
            got_any = False
            for batch in self.dataloader:
                got_any = True
                if self.global_step >= total_steps:
                    self.should_stop = True
                    break
                ev_prof.set_step(self.global_step)
                if micro % ga == 0:
                    t_host = time.perf_counter()
                    if cuda:
                        ev0 = torch.cuda.Event(enable_timing=True)
                        ev0.record()
                seqlens_acc.extend(self.batch_seqlens(batch))
                ev_prof.start("host_to_device")
                batch = send_to_device(batch, self.device)
                ev_prof.stop("host_to_device")
                if args.print_batch_input_steps and args.print_batch_input_steps > 0 and self.global_step % args.print_batch_input_steps == 0 and self.rank == 0:
                    logger.info(f"batch keys/shapes: { {k: tuple(v.shape) for k, v in batch.items() if torch.is_tensor(v)} }")
                do_step = (micro + 1) % ga == 0
                if heartbeat is not None and micro % ga == 0:
                    # between steps, on the host: learn of a failed or silent peer before launching
                    # collectives that it would never join
                    heartbeat.beat(self.global_step)
                    heartbeat.check_peers(self.global_step)
                ev_prof.start("training_step")
                try:
                    loss, grad_norm = self.training_step(batch, do_step)
                except torch.OutOfMemoryError:
                    mem_prof.dump_on_oom()
                    if heartbeat is not None:
                        heartbeat.report_error(self.global_step, "out of memory")
                    raise
                except Exception as e:
                    if heartbeat is not None:
                        heartbeat.report_error(self.global_step, f"{type(e).__name__}: {e}")
                    raise
                ev_prof.stop("training_step")
                loss_acc = loss if loss_acc is None else loss_acc + loss
                micro += 1
                if not do_step:
                    continue
                self.global_step += 1
                prof.step()
                mem_prof.step(self.global_step)
                if self.enable_perf_metrics:
                    self.count_step(seqlens_acc)
                log_now = args.logging_steps and self.global_step % max(int(args.logging_steps), 1) == 0
                if log_now or self.global_step == total_steps:
                    ev_prof.start("training_metrics")
                    if cuda:
                        ev1 = torch.cuda.Event(enable_timing=True)
                        ev1.record()
                        ev1.synchronize()
                        step_s = ev0.elapsed_time(ev1) / 1e3
                    else:
                        step_s = time.perf_counter() - t_host
                    mean_loss = loss_acc / ga
                    if self.world_size > 1:
                        mean_loss = mean_loss.clone()
                        dist.all_reduce(mean_loss, op=dist.ReduceOp.SUM)
                        mean_loss = mean_loss / self.world_size
                    self.check_device_status(heartbeat)  # the loss read below synchronises anyway
                    metrics = {"train/loss": float(mean_loss), "train/lr": args.learning_rate * self.lr_factor,
                               "train/grad_norm": float(grad_norm) if grad_norm is not None else 0.0}
                    if self.enable_perf_metrics:
                        metrics.update(self.calculate_training_metrics(seqlens_acc, step_s))
                    metrics.update(self.extra_metrics())
                    metrics["train/step_time"] = step_s
                    metrics["train/epoch"] = epoch + (micro / ga) / spe if spe else 0.0
                    ev_prof.stop("training_metrics")
                    self.log_history.append({"step": self.global_step, **metrics})
                    if self.tracking is not None:
                        self.tracking.log(metrics, step=self.global_step)
                loss_acc = None
                seqlens_acc = []
                ev_prof.flush()
                if args.save_strategy != "no" and args.save_steps and self.global_step % int(args.save_steps) == 0:
                    self.check_device_status(heartbeat)  # never write a completion marker over a failed step
                    path = self.save_checkpoints()
                    self.validation_step(path)
                self._check_eval_results()
                if self.global_step >= total_steps:
                    self.should_stop = True
                    break
            epoch += 1
            if not got_any:
                break
        prof.stop_and_save()
        mem_prof.stop()
        ev_prof.close()
        self.check_device_status(heartbeat)
        if args.save_strategy != "no" and (not args.save_steps or self.global_step % int(args.save_steps) != 0):
            self.save_checkpoints()
        if self.rank == 0:
            self.compute_tracker.save(args.output_dir)
            if self.tracking is not None:
                self.tracking.finish()
        return self.log_history
