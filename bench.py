"""Headline benchmark: Qwen2.5-7B-style dense LLM, bf16, sharded data parallel with Muon on
the 2-D weights and AdamW on the rest, 16 384 packed tokens per GPU per step (documents of
length uniform in [128, 8192], uniform random token ids, varlen attention, fused
linear + cross-entropy).  Synthetic data, random-init weights.

    python bench.py --gpus N --steps K --warmup W            # this engine
    python bench.py --impl reference --gpus N ...            # the unmodified reference

For N > 1 launch under ``python -m torch.distributed.run --nproc-per-node N``.  Rank 0 prints
ONE JSON line.  ``value`` is whole-job tokens/s timed on the device (CUDA events, max over
ranks) over exactly K optimizer steps whose inputs already sit on the device; ``e2e`` is the
same metric with, inside the timed region of every step, the pinned-host -> device copy of
that step's batch and a device -> host read of its loss, driven through the trainer's public
``training_step``.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def emit_json(obj) -> None:
    """Write the result line to the process's ORIGINAL stdout.  ``main`` points file descriptor 1 at stderr
    for the rest of the run, so banners that libraries print to stdout (NCCL's version line) cannot end up
    next to the JSON line."""
    fd = int(os.environ.get("BENCH_JSON_FD", "1"))
    os.write(fd, (json.dumps(obj) + "\n").encode())


MODEL_7B = dict(vocab_size=152064, hidden_size=3584, intermediate_size=18944, num_hidden_layers=28,
                num_attention_heads=28, num_key_value_heads=4, head_dim=128, rms_norm_eps=1e-6, rope_theta=1e6,
                tie_word_embeddings=False, attention_bias=True, initializer_range=0.02)
TOKENS_PER_GPU = 16384
METRIC = "Qwen2.5-7B FSDP2 packed tokens/s (whole job), Muon+AdamW, bf16"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.idx = device_index
        self.samples = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200", "-i", str(self.idx)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 9:
                self.samples.append(parts)

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()
        sm, smax, reasons = [], [], set()
        for p in self.samples:
            try:
                sm.append(float(p[1]))
                smax.append(float(p[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), p[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def build_config(args, out_dir):
    model_cfg = dict(MODEL_7B)
    if args.layers:
        model_cfg["num_hidden_layers"] = args.layers
    return {
        "trainer_type": "fsdp2_trainer",
        "dataset_config": {
            "dataset_type": "synthetic_packed", "dataset_format": "synthetic", "packing": True,
            "packing_strategy": "first_fit", "packing_length": args.tokens * args.sp, "data_seed": 1234,
            "extra_kwargs": {"vocab_size": model_cfg["vocab_size"], "min_len": 128, "max_len": 8192, "fill_exact": True},
        },
        "model_config": {"load_from_config": {"model_type": "qwen2", "config": model_cfg}},
        "trainer_args": dict(
            output_dir=out_dir, max_steps=10**9, learning_rate=2e-4, weight_decay=0.01, per_device_train_batch_size=1,
            bf16=True, logging_steps=10**9, save_strategy="no", lr_scheduler_type="constant", use_muon=not args.adamw,
            max_grad_norm=1.0, sharding_runtime=args.runtime, seed=0, dataloader_pin_memory=True,
            gradient_checkpointing=bool(args.checkpointing), sp_ulysses_degree=args.sp, ddp_timeout=300,
        ),
    }


def run_ours(args):
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}; launch with torch.distributed.run")
    torch.cuda.set_device(local)
    from lmms_engine_b200.launch.cli import create_train_task
    from lmms_engine_b200.ops import _cuda
    from lmms_engine_b200.ops import gemm as gemm_ops

    if args.linear_backend:
        gemm_ops.LINEAR_BACKEND = args.linear_backend
    runner = create_train_task(build_config(args, os.path.join(args.out_dir, "ours"))).build()
    tr = runner.trainer
    with torch.device("cpu"):
        pass
    tr.prepare_model()
    tr.prepare_dataloader()
    tr.prepare_optimizer()
    tr.prepare_scheduler(10**9)
    dev = tr.device
    n_steps = args.warmup + args.steps
    it = iter(tr.dataloader)
    host_batches = []
    for _ in range(2 * n_steps):
        b = next(it)
        host_batches.append({k: (v.pin_memory() if torch.is_tensor(v) else v) for k, v in b.items()})
    tokens_per_step = int(host_batches[0]["input_ids"].numel())
    h2d = sum(v.numel() * v.element_size() for v in host_batches[0].values() if torch.is_tensor(v))

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ------------------------------------------------------------ device-timed steps
    dev_batches = [{k: v.to(dev) for k, v in b.items()} for b in host_batches[:n_steps]]
    for b in dev_batches[: args.warmup]:
        tr.training_step(b, True)
    sync_all()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0 = _cuda.launch_count
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for b in dev_batches[args.warmup :]:
        tr.training_step(b, True)
    e1.record()
    sync_all()
    ms = e0.elapsed_time(e1)
    launches = _cuda.launch_count - launches0
    clocks = sampler.stop() if rank == 0 else None
    _cuda.check_status()
    del dev_batches

    # ------------------------------------------------------------ end to end (H2D + loss read-back per step)
    e2e_batches = host_batches[n_steps:]
    for b in e2e_batches[: args.warmup]:
        loss, _ = tr.training_step({k: v.to(dev, non_blocking=True) for k, v in b.items()}, True)
        float(loss)
    sync_all()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    last = None
    for b in e2e_batches[args.warmup :]:
        loss, _ = tr.training_step({k: v.to(dev, non_blocking=True) for k, v in b.items()}, True)
        last = float(loss)  # 4-byte device -> host read, synchronises the step
    t1.record()
    sync_all()
    ms_e2e = t0.elapsed_time(t1)

    t = torch.tensor([ms, ms_e2e], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, ms_e2e = float(t[0]), float(t[1])
    peak_gb = torch.cuda.max_memory_allocated() / 2**30
    if rank == 0:
        total_tokens = tokens_per_step * (world // args.sp) * args.steps  # one packed sequence per sequence-parallel group
        value = total_tokens / (ms / 1e3)
        e2e = total_tokens / (ms_e2e / 1e3)
        seqlens = (host_batches[0]["cu_seqlens"][1:] - host_batches[0]["cu_seqlens"][:-1]).tolist()
        flops = tr.flops_counter.flops_per_step(seqlens)
        out = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic (uniform random ids, docs U[128,8192] packed to 16384 tokens/GPU), random-init weights",
            "config": {"model": "Qwen2.5-7B-style (28L, h3584, 28q/4kv, d128, ffn18944, vocab152064, qkv bias)",
                       "global_batch": tokens_per_step * (world // args.sp), "seq_len": tokens_per_step,
                       "parallelism": (f"dp{world} ({tr.runtime_kind} runtime)" if args.sp == 1 else
                                       f"dp{world // args.sp} x ulysses{args.sp} ({tr.runtime_kind} runtime; not the headline layout)"), "optimizer": "adamw" if args.adamw else "muon+adamw",
                       "l2": "inputs and weights larger than L2 every step (15 GB of parameters)",
                       "layers": build_config(args, "x")["model_config"]["load_from_config"]["config"]["num_hidden_layers"],
                       "linear_backend": gemm_ops.LINEAR_BACKEND, "gradient_checkpointing": bool(args.checkpointing)},
            "clocks": clocks, "e2e": {"value": e2e, "unit": "tokens/s", "ms_per_step": ms_e2e / args.steps,
                                      "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4},
            "gpu_launches": launches, "tokens_per_gpu_per_s": value / world,
            "mfu_ref_formula": flops / (ms / args.steps / 1e3) / 2.25e15, "peak_mem_gb": peak_gb, "last_loss": last,
        }
        emit_json(out)
    if dist.is_initialized():
        dist.destroy_process_group()


def run_reference(args):
    from baseline.reference_arm import run as run_ref

    run_ref(args)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--tokens", type=int, default=TOKENS_PER_GPU)
    ap.add_argument("--layers", type=int, default=0, help="debug: fewer layers (invalidates the number)")
    ap.add_argument("--adamw", action="store_true", help="AdamW only (not the headline config)")
    ap.add_argument("--runtime", default="native", choices=["native", "native_sharded", "torch_fsdp2", "auto"])
    ap.add_argument("--linear-backend", default=None, choices=[None, "tcgen05", "cublas"])
    ap.add_argument("--checkpointing", type=int, default=0,
                    help="gradient checkpointing, the same setting for both arms")
    ap.add_argument("--sp", type=int, default=1, help="Ulysses degree (not the headline layout; sequence = tokens * sp)")
    ap.add_argument("--out-dir", default=os.path.join(tempfile.gettempdir(), "lmms_engine_b200_bench"),
                    help="trainer output directory (nothing is saved there during the timed steps)")
    args = ap.parse_args()
    sys.stdout.flush()
    os.environ["BENCH_JSON_FD"] = str(os.dup(1))
    os.dup2(2, 1)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
