"""Times the unmodified reference (installed under ``baseline/_ref``) on the headline
configuration: Qwen2.5-7B-style model from ``load_from_config``, its ``fsdp2_trainer``
(FSDP2 + rmpad + Liger + flash-attention as in its own ``examples/qwen2_5_llm`` config),
synthetic packed batches of 16 384 tokens per GPU.

What is NOT the reference's code here, and why:
* the stand-in modules of ``baseline/shims`` for third-party packages missing from this
  offline image (none of them on the timed path),
* a synthetic dataset registered through the reference's own ``@register_dataset`` hook and
  a collator that emits the reference's padded batch contract,
* for the Muon configuration, a ``prepare_optimizer`` override registered through the
  reference's ``TRAINER_REGISTER`` that instantiates the reference's own ``Muon`` class with
  the parameter grouping of its HF trainer: the reference wires Muon only into its
  accelerate-based trainer, which cannot be constructed without accelerate.
The timed region calls the reference trainer's own ``training_step`` (forward, backward,
clip, optimizer, scheduler, its loss all-reduce and ``.item()`` reads) exactly K times.
"""
from __future__ import annotations

import json
import os


def _emit(obj) -> None:
    """Result line on the descriptor that ``bench.py`` kept for it (its original stdout)."""
    os.write(int(os.environ.get("BENCH_JSON_FD", "1")), (json.dumps(obj) + "\n").encode())
import statistics
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)

MODEL_7B = dict(vocab_size=152064, hidden_size=3584, intermediate_size=18944, num_hidden_layers=28,
                num_attention_heads=28, num_key_value_heads=4, rms_norm_eps=1e-6, rope_theta=1e6,
                tie_word_embeddings=False, max_position_embeddings=32768, initializer_range=0.02)


def _prepare_imports():
    from baseline.shims.install_shims import install_all

    install_all()
    for k in [k for k in sys.modules if k == "lmms_engine" or k.startswith("lmms_engine.")]:
        del sys.modules[k]
    sys.path[:] = [p for p in sys.path if os.path.abspath(p or ".") != ROOT]
    sys.path.insert(0, os.path.join(HERE, "_ref"))


def _assert_patched(model) -> None:
    """The reference swallows every error of its monkey-patch step and carries on with the
    plain ``transformers`` model on padded batches with full logits
    (``train/runner.py:113-126``).  A number from that state is not the reference's
    rmpad + Liger configuration, so this arm refuses to time it: the checks below look at the
    reference's own objects after ``runner.build()``
    (``models/qwen2/monkey_patch.py:62-93``)."""
    from liger_kernel.transformers.rms_norm import LigerRMSNorm
    from liger_kernel.transformers.swiglu import LigerSwiGLUMLP
    from lmms_engine.models.qwen2 import qwen2_ops
    from transformers.models.qwen2 import modeling_qwen2 as mq

    problems = []
    if mq.Qwen2Model.forward is not qwen2_ops.model_forward:
        problems.append("Qwen2Model.forward is not the reference's rmpad model_forward")
    if mq.Qwen2DecoderLayer.forward is not qwen2_ops.decoder_layer_forward:
        problems.append("Qwen2DecoderLayer.forward is not the reference's rmpad decoder_layer_forward")
    if mq.Qwen2Attention.forward is not qwen2_ops.attn_forward:
        problems.append("Qwen2Attention.forward is not the reference's rmpad attn_forward")
    fwd = mq.Qwen2ForCausalLM.forward
    if getattr(getattr(fwd, "__wrapped__", fwd), "__name__", "") != "qwen2_lce_forward":
        problems.append("Qwen2ForCausalLM.forward is not the reference's qwen2_lce_forward (fused linear + CE)")
    layer = model.model.layers[0]
    if layer.mlp.forward.__func__ is not LigerSwiGLUMLP.forward:
        problems.append("decoder MLP instances do not run LigerSwiGLUMLP.forward")
    if layer.input_layernorm.forward.__func__ is not LigerRMSNorm.forward:
        problems.append("RMSNorm instances do not run LigerRMSNorm.forward")
    if problems:
        raise RuntimeError("reference rmpad/Liger patch did not apply: " + "; ".join(problems))


def _transformers_compat(model) -> None:
    """The reference's rmpad forward reads ``decoder_layer.attention_type``
    (``models/qwen2/qwen2_ops.py:152``), an attribute that ``transformers`` 4.5x set on every
    ``Qwen2DecoderLayer`` and that the installed 5.x no longer sets (it indexes
    ``config.layer_types`` instead), although the reference declares ``transformers < 5.9`` as
    supported.  The attribute is restored on the model instance, with the value the older
    library gave it, so that the reference's own code runs unchanged."""
    cfg = model.config
    types = getattr(cfg, "layer_types", None) or ["full_attention"] * cfg.num_hidden_layers
    for i, layer in enumerate(model.model.layers):
        if not hasattr(layer, "attention_type"):
            layer.attention_type = types[i]


def main(args):
    import numpy as np
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    sys.path.insert(0, ROOT)
    from bench import ClockSampler, METRIC

    _prepare_imports()
    import lmms_engine  # the reference package

    assert os.path.abspath(lmms_engine.__file__).startswith(os.path.join(HERE, "_ref")), lmms_engine.__file__
    from lmms_engine.launch.cli import create_train_task
    from lmms_engine.mapping_func import register_dataset
    from lmms_engine.train import TRAINER_REGISTER
    from lmms_engine.train.fsdp2.fsdp2_trainer import FSDP2SFTTrainer

    tokens = args.tokens
    vocab = MODEL_7B["vocab_size"]

    class _PadCollator:
        """The reference's batch contract: ``input_ids/labels [n_docs, L]`` + ``attention_mask``."""

        def __call__(self, batch):
            docs = [d for pack in batch for d in pack]
            L = max(d["input_ids"].numel() for d in docs)
            ids = torch.zeros(len(docs), L, dtype=torch.long)
            lab = torch.full((len(docs), L), -100, dtype=torch.long)
            am = torch.zeros(len(docs), L, dtype=torch.long)
            for i, d in enumerate(docs):
                n = d["input_ids"].numel()
                ids[i, :n] = d["input_ids"]
                lab[i, :n] = d["labels"]
                am[i, :n] = 1
            return {"input_ids": ids, "labels": lab, "attention_mask": am}

    @register_dataset("synthetic_packed_bench")
    class SyntheticPacked(torch.utils.data.IterableDataset):
        def __init__(self, config):
            self.config = config
            self.processor = None

        def build(self):
            return self

        def get_collator(self):
            return _PadCollator()

        def __iter__(self):
            idx = 0
            buf, used = [], 0
            while True:
                rng = np.random.default_rng([1234, rank, idx])
                idx += 1
                n = int(rng.integers(128, 8193))
                ids = torch.from_numpy(rng.integers(0, vocab, size=n, dtype=np.int64))
                room = tokens - used
                if n >= room:
                    buf.append({"input_ids": ids[:room], "labels": ids[:room].clone()})
                    yield buf
                    buf, used = [], 0
                else:
                    buf.append({"input_ids": ids, "labels": ids.clone()})
                    used += n

    if not args.adamw:

        @TRAINER_REGISTER.register("fsdp2_trainer_muon_bench")
        class FSDP2Muon(FSDP2SFTTrainer):
            def prepare_optimizer(self):
                from lmms_engine.utils.muon_utils import Muon

                exclude = ["emb", "norm", "lm_head", "bias", "wte", "wpe", "output", "a_proj", "b_proj", "conv1d", "rotary"]
                mu, ad = [], []
                for name, p in self.fsdp2_model.named_parameters():
                    if not p.requires_grad:
                        continue
                    (mu if (p.ndim == 2 and not any(e in name for e in exclude)) else ad).append(p)
                groups = [
                    dict(params=mu, use_muon=True, lr=self.args.learning_rate, weight_decay=self.args.weight_decay),
                    dict(params=ad, use_muon=False, lr=self.args.learning_rate, weight_decay=self.args.weight_decay,
                         betas=(self.args.adam_beta1, self.args.adam_beta2), eps=self.args.adam_epsilon),
                ]
                self.optimizer = Muon(groups)

    model_cfg = dict(MODEL_7B)
    if args.layers:
        model_cfg["num_hidden_layers"] = args.layers
    out_dir = os.path.join(args.out_dir, "reference")
    cfg = {
        "trainer_type": "fsdp2_trainer" if args.adamw else "fsdp2_trainer_muon_bench",
        "dataset_config": {"dataset_type": "synthetic_packed_bench", "dataset_format": "json", "processor_config": {"processor_name": "none", "processor_type": "pure_text"},
                           "packing": True, "packing_strategy": "first_fit", "packing_length": tokens},
        "model_config": {"load_from_config": {"model_type": "qwen2", "config": model_cfg}, "attn_implementation": "flash_attention_2",
                         "extra_kwargs": {"torch_dtype": torch.bfloat16, "attn_implementation": "flash_attention_2"}},
        "trainer_args": dict(
            output_dir=out_dir, max_steps=10**6, learning_rate=2e-4, weight_decay=0.01, per_device_train_batch_size=1,
            bf16=True, logging_steps=10**6, save_strategy="no", lr_scheduler_type="constant", max_grad_norm=1.0,
            use_liger_kernel=True, use_rmpad=True, fsdp2=True, gradient_checkpointing=bool(args.checkpointing),
            fsdp_config={"transformer_layer_cls_to_wrap": ["Qwen2DecoderLayer"], "reshard_after_forward": False},
            report_to="none", seed=0, dataloader_pin_memory=True, dataloader_num_workers=0,
        ),
    }
    runner = create_train_task(cfg)
    runner.build()
    _assert_patched(runner.model)
    _transformers_compat(runner.model)
    tr = runner.trainer
    tr.prepare_model()
    loader = tr.prepare_dataloader(tr.train_dataset, is_training=True)
    tr.train_dataloader = loader
    tr.prepare_optimizer()
    tr.total_steps = 10**6
    tr.prepare_scheduler(0, 10**6)
    tr.global_step = 0
    try:
        tr.ema.maybe_init(model=tr.fsdp2_model, checkpoint_dir=None)
    except Exception:
        pass
    dev = torch.device("cuda", local)
    n_steps = args.warmup + args.steps
    it = iter(loader)
    host = []
    for _ in range(2 * n_steps):
        b = next(it)
        host.append({k: v.pin_memory() for k, v in b.items()})
    h2d = sum(v.numel() * v.element_size() for v in host[0].values())

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    dev_batches = [{k: v.to(dev) for k, v in b.items()} for b in host[:n_steps]]
    for b in dev_batches[: args.warmup]:
        tr.training_step(b)
    sync_all()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for b in dev_batches[args.warmup :]:
        tr.training_step(b)
    e1.record()
    sync_all()
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop() if rank == 0 else None
    del dev_batches
    for b in host[n_steps : n_steps + args.warmup]:
        tr.training_step({k: v.to(dev, non_blocking=True) for k, v in b.items()})
    sync_all()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    last = None
    for b in host[n_steps + args.warmup :]:
        m = tr.training_step({k: v.to(dev, non_blocking=True) for k, v in b.items()})
        last = m.get("train/loss")  # already read back on the host by the reference's step
    t1.record()
    sync_all()
    ms_e2e = t0.elapsed_time(t1)
    t = torch.tensor([ms, ms_e2e], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, ms_e2e = float(t[0]), float(t[1])
    if rank == 0:
        total = tokens * world * args.steps
        _emit({
            "impl": "reference", "metric": METRIC, "value": total / (ms / 1e3), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic (uniform random ids, docs U[128,8192] packed to 16384 tokens/GPU), random-init weights",
            "config": {"model": "Qwen2.5-7B-style via transformers Qwen2ForCausalLM + reference rmpad/Liger patches",
                       "global_batch": tokens * world, "seq_len": tokens, "parallelism": f"dp{world} (reference fsdp2_trainer, FSDP2)",
                       "optimizer": "adamw" if args.adamw else "muon+adamw (reference Muon class)",
                       "gradient_checkpointing": bool(args.checkpointing), "layers": model_cfg["num_hidden_layers"]},
            "clocks": clocks,
            "e2e": {"value": total / (ms_e2e / 1e3), "unit": "tokens/s", "ms_per_step": ms_e2e / args.steps,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 8},
            "peak_mem_gb": torch.cuda.max_memory_allocated() / 2**30, "last_loss": last,
        })
    if dist.is_initialized():
        dist.destroy_process_group()
