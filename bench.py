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


QWEN25_VIT = dict(depth=32, hidden_size=1280, intermediate_size=3420, num_heads=16, patch_size=14, temporal_patch_size=2,
                  spatial_merge_size=2, in_channels=3, window_size=112, fullatt_block_indexes=[7, 15, 23, 31], out_hidden_size=3584)
QWEN3_VIT = dict(depth=27, hidden_size=1152, intermediate_size=4304, num_heads=16, patch_size=16, temporal_patch_size=2,
                 spatial_merge_size=2, in_channels=3, out_hidden_size=4096, num_position_embeddings=2304,
                 deepstack_visual_indexes=[8, 16, 24])
QWEN3_MOE_30B = dict(vocab_size=151936, hidden_size=2048, intermediate_size=6144, num_hidden_layers=48, num_attention_heads=32,
                     num_key_value_heads=4, head_dim=128, rms_norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=False,
                     num_experts=128, num_experts_per_tok=8, moe_intermediate_size=768, decoder_sparse_step=1, norm_topk_prob=True,
                     mlp_only_layers=[], router_aux_loss_coef=1e-3, initializer_range=0.02)
QWEN3_VL_8B_TEXT = dict(vocab_size=151936, hidden_size=4096, intermediate_size=12288, num_hidden_layers=36, num_attention_heads=32,
                        num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-6, rope_theta=5e6, tie_word_embeddings=False,
                        initializer_range=0.02)

# The configurations of BASELINE.json beyond the headline one.  Each names its nominal layout on 8 GPUs; with fewer
# GPUs the model-parallel degree shrinks to what fits (a debugging aid, reported as such in the JSON line).
CONFIGS = {
    "qwen2_5_7b": dict(metric=METRIC, tokens=TOKENS_PER_GPU),
    "vl_sp8": dict(metric="Qwen2.5-VL-7B Ulysses-8 packed tokens/s (whole job), 65536-token samples, AdamW, bf16", tokens=65536, sp=8),
    "moe_ep8": dict(metric="Qwen3-30B-A3B expert-parallel-8 packed tokens/s (whole job), AdamW, bf16", tokens=8192, ep=8),
    "vl_tp4": dict(metric="Qwen3-VL-8B TP4 x FSDP2 packed tokens/s (whole job), 32768-token video samples, AdamW, bf16", tokens=32768, tp=4),
}


def resolve_layout(args):
    """Model-parallel degrees for this run: the configuration's nominal degree, reduced to the largest divisor
    of the world size when fewer GPUs are used than the configuration names."""
    c = CONFIGS[args.config]
    world = args.gpus

    def fit(n):
        n = min(n, world)
        while world % n:
            n -= 1
        return n

    sp = fit(c.get("sp", args.sp))
    tp = fit(c.get("tp", 1))
    ep = fit(c.get("ep", 1))
    return sp, tp, ep


def build_config(args, out_dir):
    sp, tp, ep = resolve_layout(args)
    tokens = args.tokens or CONFIGS[args.config]["tokens"]
    targs = dict(
        output_dir=out_dir, max_steps=10**9, learning_rate=2e-4, weight_decay=0.01, per_device_train_batch_size=1,
        bf16=True, logging_steps=10**9, save_strategy="no", lr_scheduler_type="constant", use_muon=not args.adamw,
        max_grad_norm=1.0, sharding_runtime=args.runtime, seed=0, dataloader_pin_memory=True,
        gradient_checkpointing=bool(args.checkpointing), sp_ulysses_degree=sp, tp_degree=tp, ep_degree=ep, ddp_timeout=300,
    )
    if args.config == "qwen2_5_7b":
        model_cfg = dict(MODEL_7B)
        if args.layers:
            model_cfg["num_hidden_layers"] = args.layers
        return {
            "trainer_type": "fsdp2_trainer",
            "dataset_config": {
                "dataset_type": "synthetic_packed", "dataset_format": "synthetic", "packing": True,
                "packing_strategy": "first_fit", "packing_length": tokens * sp, "data_seed": 1234,
                "extra_kwargs": {"vocab_size": model_cfg["vocab_size"], "min_len": 128, "max_len": 8192, "fill_exact": True},
            },
            "model_config": {"load_from_config": {"model_type": "qwen2", "config": model_cfg}},
            "trainer_args": targs,
        }
    targs["use_muon"] = False  # BASELINE names Muon only for the dense headline configuration
    if args.config == "moe_ep8":
        model_cfg = dict(QWEN3_MOE_30B)
        if args.layers:
            model_cfg["num_hidden_layers"] = args.layers
        targs["sharding_runtime"] = "auto"  # expert parallelism composes with stock FSDP2 (parallel/plans.py)
        return {
            "trainer_type": "fsdp2_trainer",
            "dataset_config": {
                "dataset_type": "synthetic_packed", "dataset_format": "synthetic", "packing": True,
                "packing_strategy": "first_fit", "packing_length": tokens, "data_seed": 1234,
                "extra_kwargs": {"vocab_size": model_cfg["vocab_size"], "min_len": 128, "max_len": 4096, "fill_exact": True},
            },
            "model_config": {"load_from_config": {"model_type": "qwen3_moe", "config": model_cfg}},
            "trainer_args": targs,
        }
    if args.config == "vl_sp8":
        text = dict(MODEL_7B, rope_scaling={"type": "mrope", "mrope_section": [16, 24, 24]})
        vis = dict(QWEN25_VIT)
        if args.layers:
            text["num_hidden_layers"] = args.layers
            vis["depth"] = max(4, args.layers)
            vis["fullatt_block_indexes"] = [vis["depth"] - 1]
        data = dict(vocab_size=text["vocab_size"], media="image", num_media=[4, 16], size=[448, 1344], size_multiple=28,
                    patch_size=14, temporal_patch_size=2, merge_size=2, image_token_id=151655, video_token_id=151656)
        model = dict(model_type="qwen2_5_vl", text_config=text, vision_config=vis, image_token_id=151655, video_token_id=151656)
        mtype = "qwen2_5_vl"
    else:  # vl_tp4
        text = dict(QWEN3_VL_8B_TEXT, rope_scaling={"mrope_section": [24, 20, 20], "mrope_interleaved": True})
        vis = dict(QWEN3_VIT)
        if args.layers:
            text["num_hidden_layers"] = args.layers
            vis["depth"] = max(4, args.layers)
            vis["deepstack_visual_indexes"] = [0, 1, 2]
        data = dict(vocab_size=text["vocab_size"], media="video", num_media=[1, 1], size=[448, 768], size_multiple=32, frames=[32, 64],
                    patch_size=16, temporal_patch_size=2, merge_size=2, image_token_id=151655, video_token_id=151656)
        model = dict(model_type="qwen3_vl", text_config=text, vision_config=vis, image_token_id=151655, video_token_id=151656)
        mtype = "qwen3_vl"
        targs["sharding_runtime"] = "auto"  # tensor parallelism composes with stock FSDP2
    return {
        "trainer_type": "fsdp2_trainer",
        "dataset_config": {"dataset_type": "synthetic_vl", "dataset_format": "synthetic", "packing": True,
                           "packing_length": tokens, "data_seed": 1234, "extra_kwargs": data},
        "model_config": {"load_from_config": {"model_type": mtype, "config": model},
                         # frames are balanced over the ranks of the native runtime; under tensor parallelism the tower is
                         # an FSDP2 unit that every rank runs on its own sample (as in the reference)
                         "monkey_patch_kwargs": {"vit_frame_parallel": args.gpus > 1 and args.config == "vl_sp8"}},
        "trainer_args": targs,
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
    sp, tp, ep = resolve_layout(args)
    replicas = world // (sp * tp)  # independent token streams per step
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

    # LMMS_B200_STEP_BREAKDOWN=1: exposed device time of every phase of one more step (max over ranks)
    breakdown = None
    if tr.runtime is not None and getattr(tr.runtime, "breakdown", False):
        tr.training_step({k: v.to(dev) for k, v in host_batches[0].items()}, True)
        phases = tr.runtime.phase_times()
        names = sorted(phases)
        pt = torch.tensor([phases[n] for n in names], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(pt, op=dist.ReduceOp.MAX)
        breakdown = {n: round(float(v), 3) for n, v in zip(names, pt)}

    t = torch.tensor([ms, ms_e2e], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, ms_e2e = float(t[0]), float(t[1])
    peak_gb = torch.cuda.max_memory_allocated() / 2**30
    # peer-mapped (symmetric) buffers are allocated outside torch's caching allocator
    symm_gb = getattr(getattr(tr.runtime, "comm", None), "allocated_bytes", 0) / 2**30 if tr.runtime is not None else 0.0
    if rank == 0:
        total_tokens = tokens_per_step * replicas * args.steps  # one packed sequence per model-parallel group
        value = total_tokens / (ms / 1e3)
        e2e = total_tokens / (ms_e2e / 1e3)
        seqlens = (host_batches[0]["cu_seqlens"][1:] - host_batches[0]["cu_seqlens"][:-1]).tolist()
        flops = tr.flops_counter.flops_per_step(seqlens) / (sp * tp)  # the reference's MFU: model FLOPs per rank of a model-parallel group
        cfg_now = build_config(args, "x")
        mc = cfg_now["model_config"]["load_from_config"]["config"]
        layers = (mc.get("text_config") or mc)["num_hidden_layers"]
        nominal = CONFIGS[args.config]
        layout = "dp%d" % replicas + (f" x ulysses{sp}" if sp > 1 else "") + (f" x tp{tp}" if tp > 1 else "") + (f", ep{ep}" if ep > 1 else "")
        reduced = any(nominal.get(k, 1) != v for k, v in (("sp", sp), ("tp", tp), ("ep", ep)) if k in nominal) or bool(args.layers)
        descr = {"qwen2_5_7b": "Qwen2.5-7B-style (28L, h3584, 28q/4kv, d128, ffn18944, vocab152064, qkv bias)",
                 "vl_sp8": "Qwen2.5-VL-7B-style (32L ViT h1280 p14 window+full attention, 2x2 merge; 7B decoder, sectioned M-RoPE)",
                 "moe_ep8": "Qwen3-30B-A3B-style (48L, h2048, 32q/4kv, QK-norm, 128 experts top-8, expert ffn 768, aux loss 1e-3)",
                 "vl_tp4": "Qwen3-VL-8B-style (27L ViT h1152 p16 deepstack; 36L h4096 32q/8kv decoder, interleaved M-RoPE)"}[args.config]
        data_descr = {"qwen2_5_7b": "synthetic (uniform random ids, docs U[128,8192] packed to 16384 tokens/GPU), random-init weights",
                      "vl_sp8": "synthetic (4-16 images of 448-1344 px, N(0,1) pixels, text spans of uniform random ids, 65536-token samples, loss on text), random-init weights",
                      "moe_ep8": "synthetic (uniform random ids, docs U[128,4096] packed to 8192 tokens/GPU), random-init weights",
                      "vl_tp4": "synthetic (one 32-64 frame video of 448-768 px per sample, N(0,1) pixels, uniform random text, 32768-token samples, loss on text), random-init weights"}[args.config]
        out = {
            "metric": nominal["metric"], "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": data_descr,
            "config": {"name": args.config, "model": descr,
                       "global_batch": tokens_per_step * replicas, "seq_len": tokens_per_step,
                       "parallelism": f"{layout} ({tr.runtime_kind} runtime" + ("; reduced from the named layout)" if reduced else ")"),
                       "optimizer": "muon+adamw" if cfg_now["trainer_args"]["use_muon"] else "adamw",
                       "l2": "inputs and weights larger than L2 every step",
                       "layers": layers,
                       "linear_backend": gemm_ops.LINEAR_BACKEND, "gradient_checkpointing": bool(args.checkpointing)},
            "clocks": clocks, "e2e": {"value": e2e, "unit": "tokens/s", "ms_per_step": ms_e2e / args.steps,
                                      "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4},
            "gpu_launches": launches, "tokens_per_gpu_per_s": value / world,
            "mfu_ref_formula": flops / (ms / args.steps / 1e3) / 2.25e15, "peak_mem_gb": peak_gb + symm_gb, "peak_mem_allocator_gb": peak_gb,
            "peer_mapped_mem_gb": symm_gb, "last_loss": last,
        }
        if breakdown is not None:
            out["step_breakdown_ms"] = breakdown
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
    ap.add_argument("--config", default="qwen2_5_7b", choices=sorted(CONFIGS),
                    help="qwen2_5_7b is the headline configuration; the others are the further BASELINE configurations")
    ap.add_argument("--tokens", type=int, default=0, help="tokens per GPU (per sample for the multimodal configurations); 0 = the configuration's")
    ap.add_argument("--layers", type=int, default=0, help="debug: fewer layers (invalidates the number)")
    ap.add_argument("--adamw", action="store_true", help="AdamW only (not the headline config)")
    ap.add_argument("--runtime", default="default", choices=["default", "native", "native_sharded", "torch_fsdp2", "auto"],
                    help="default: the headline configuration on several GPUs shards the block parameters (native_sharded: "
                         "979 vs 1008 ms / step on 4 GPUs, 13 GB less); one GPU and the other configurations run 'native'")
    ap.add_argument("--linear-backend", default=None, choices=[None, "tcgen05", "cublas"])
    ap.add_argument("--checkpointing", type=int, default=0,
                    help="gradient checkpointing, the same setting for both arms")
    ap.add_argument("--sp", type=int, default=1, help="Ulysses degree (not the headline layout; sequence = tokens * sp)")
    ap.add_argument("--out-dir", default=os.path.join(tempfile.gettempdir(), "lmms_engine_b200_bench"),
                    help="trainer output directory (nothing is saved there during the timed steps)")
    args = ap.parse_args()
    if args.runtime == "default":
        args.runtime = "native_sharded" if (args.gpus > 1 and args.config == "qwen2_5_7b" and args.sp == 1) else "native"
    sys.stdout.flush()
    os.environ["BENCH_JSON_FD"] = str(os.dup(1))
    os.dup2(2, 1)
    if args.impl == "reference" and args.config != "qwen2_5_7b":
        from baseline.reference_arm import unavailable

        why = {"vl_sp8": "the reference requires num_heads % sp_ulysses_degree == 0 (parallel/sequence_parallel/ulysses.py:445-449): "
                         "28 query heads cannot be split over 8 ranks",
               }.get(args.config, "the reference arm of this build drives the headline configuration only")
        unavailable(f"{args.config}: {why}")
    elif args.impl == "reference":
        if not args.tokens:
            args.tokens = TOKENS_PER_GPU
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
