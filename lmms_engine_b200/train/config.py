"""Trainer configuration.

``TrainingArguments`` carries the Hugging Face argument names the engine consumes plus the
engine extras of the reference (src/lmms_engine/train/config.py:10-56).  It is a plain
dataclass: the reference subclasses ``transformers.TrainingArguments``, which needs
``accelerate`` at construction; here unknown HF keys are accepted by ``filter_training_args``
(launch/cli.py) and dropped with a warning, exactly like unsupported keys upstream.
"""
from __future__ import annotations

import dataclasses
from dataclasses import asdict, dataclass, field
from typing import Any, Dict, List, Literal, Optional

from ..datasets.config import DatasetConfig
from ..models.config import ModelConfig


@dataclass
class TrainingArguments:
    # ---- Hugging Face names -------------------------------------------------------------
    output_dir: str = "./output"
    overwrite_output_dir: bool = False
    per_device_train_batch_size: int = 1
    per_device_eval_batch_size: int = 1
    gradient_accumulation_steps: int = 1
    learning_rate: float = 5e-5
    weight_decay: float = 0.0
    adam_beta1: float = 0.9
    adam_beta2: float = 0.999
    adam_epsilon: float = 1e-8
    max_grad_norm: float = 1.0
    num_train_epochs: float = 1.0
    max_steps: int = -1
    lr_scheduler_type: str = "cosine"
    lr_scheduler_kwargs: Optional[Dict[str, Any]] = None
    warmup_ratio: float = 0.0
    warmup_steps: int = 0
    logging_steps: int = 1
    logging_dir: Optional[str] = None
    save_strategy: str = "steps"
    save_steps: int = 500
    save_total_limit: Optional[int] = None
    save_only_model: bool = False
    seed: int = 42
    data_seed: Optional[int] = None
    bf16: bool = False
    fp16: bool = False
    tf32: Optional[bool] = None
    gradient_checkpointing: bool = False
    gradient_checkpointing_kwargs: Optional[Dict[str, Any]] = None
    dataloader_num_workers: int = 0
    dataloader_drop_last: bool = False
    dataloader_pin_memory: bool = True
    dataloader_prefetch_factor: Optional[int] = None
    remove_unused_columns: bool = False
    report_to: Any = "none"
    run_name: Optional[str] = None
    use_cpu: bool = False
    ddp_timeout: int = 1800
    fsdp: Any = ""
    fsdp_config: Optional[Dict[str, Any]] = None
    deepspeed: Optional[str] = None
    use_liger_kernel: bool = False
    torch_compile: bool = False
    optim: str = "adamw_torch"
    eval_strategy: str = "no"
    eval_steps: Optional[int] = None
    resume_from_checkpoint: Optional[str] = None
    average_tokens_across_devices: bool = False
    # ---- engine extras ------------------------------------------------------------------
    use_muon: Optional[bool] = False
    freeze_modules: Optional[List[str]] = None
    use_rmpad: Optional[bool] = False
    fsdp2: Optional[bool] = False
    reduce_dtype: Optional[str] = "bfloat16"
    output_dtype: Optional[str] = "bfloat16"
    print_batch_input_steps: Optional[int] = -1
    enable_profiler: Optional[bool] = False
    profiler_config: Optional[Dict[str, Any]] = None
    enable_memory_snapshot: Optional[bool] = False
    memory_snapshot_config: Optional[Dict[str, Any]] = None
    enable_cuda_event_profiler: Optional[bool] = False
    # > 0: ranks publish a heartbeat in the process group's store between steps and stop with a clear
    # error when a peer reported a failure or stayed silent for this many seconds
    heartbeat_timeout: float = 0.0
    cuda_event_profiler_config: Optional[Dict[str, Any]] = None
    ep_degree: Optional[int] = 1
    sp_ulysses_degree: Optional[int] = 1
    tp_degree: Optional[int] = 1
    ema_enabled: Optional[bool] = False
    ema_decay: Optional[float] = 0.9999
    ema_update_every: Optional[int] = 1
    ema_start_step: Optional[int] = 0
    ema_requires_grad_only: Optional[bool] = True
    ema_param_filter: Optional[Dict[str, Any]] = None
    ema_resume_from_ema: Optional[bool] = False
    eval_config: Optional[Dict[str, Any]] = None
    carbon_intensity: Optional[float] = 0.475
    group_by_length: Optional[bool] = False
    only_save_mm_adapter: Optional[bool] = False
    # Muon hyper-parameters (the reference hard-codes momentum 0.95 / 5 Newton-Schulz steps)
    muon_momentum: float = 0.95
    muon_ns_steps: int = 5
    muon_nesterov: bool = True
    # RL (GRPO) trainer
    rl_config: Optional[Dict[str, Any]] = None
    # RAE trainer: perceptual / adversarial recipe (keys and defaults: train/fsdp2/extra_trainers.py GAN_DEFAULTS)
    gan_config: Optional[Dict[str, Any]] = None
    # engine runtime: "auto" picks the native sharded runtime on CUDA and stock FSDP2 on CPU
    sharding_runtime: str = "auto"

    def __post_init__(self):
        if self.fsdp_config is None:
            self.fsdp_config = {}
        if self.lr_scheduler_kwargs is None:
            self.lr_scheduler_kwargs = {}
        if self.bf16 and self.fp16:
            raise ValueError("bf16 and fp16 are mutually exclusive")

    @classmethod
    def field_names(cls):
        return {f.name for f in dataclasses.fields(cls)}

    def to_dict(self) -> Dict[str, Any]:
        return asdict(self)

    @property
    def process_index(self) -> int:
        import torch.distributed as dist

        return dist.get_rank() if dist.is_available() and dist.is_initialized() else 0

    @property
    def world_size(self) -> int:
        import torch.distributed as dist

        return dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1


@dataclass
class TrainerConfig:
    trainer_type: str
    dataset_config: DatasetConfig
    trainer_args: TrainingArguments
    model_config: ModelConfig
    extra_kwargs: Dict[str, Any] = None

    def to_dict(self):
        return {
            "trainer_type": self.trainer_type,
            "dataset_config": self.dataset_config.to_dict(),
            "trainer_args": self.trainer_args.to_dict(),
            "model_config": self.model_config.to_dict(),
            "extra_kwargs": self.extra_kwargs,
        }
