"""Training smoke suite: every model family takes a few optimizer steps under ``torch.distributed.run`` through the
public command line (``python -m lmms_engine_b200.launch.cli config_yaml=...``) on a tiny random-init model and
synthetic data, and must exit 0 with finite losses in its log.

The role of test/train/run_cicd.py + cicd/run_traincicd.sh of the reference (one ``torchrun`` per family on all visible
GPUs, return code 0 is the assertion), without its hub download: nothing is read from disk but the YAML written here.

    python tests/train/run_cicd.py --gpu-count 2                  # every family on 2 GPUs (NCCL)
    python tests/train/run_cicd.py --model-name qwen3_moe --cpu   # one family on 2 CPU ranks (gloo)
"""
from __future__ import annotations

import argparse
import json
import math
import os
import re
import socket
import subprocess
import sys
import tempfile
import time
from typing import Dict, List, Optional

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

# small, but of shapes the tensor-core kernels take (hidden sizes in multiples of 128, head sizes of 32 and 64)
LM = dict(vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
          head_dim=32, rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=1024)
MOE = dict(LM, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=128, norm_topk_prob=True, router_aux_loss_coef=0.001)
HYBRID = dict(LM, num_hidden_layers=4, head_dim=64, linear_conv_kernel_dim=4, linear_key_head_dim=32, linear_value_head_dim=32,
              linear_num_key_heads=2, linear_num_value_heads=4, rope_parameters={"rope_theta": 10000.0, "partial_rotary_factor": 0.25})
VL_TEXT = dict(LM, rope_scaling={"mrope_section": [8, 4, 4], "mrope_interleaved": True})
VISION = dict(depth=2, hidden_size=128, intermediate_size=256, num_heads=4, patch_size=8, temporal_patch_size=2, spatial_merge_size=2,
              out_hidden_size=128, num_position_embeddings=16, deepstack_visual_indexes=[0, 1], in_channels=3)


def _packed(vocab: int = 512) -> dict:
    return {"dataset_type": "synthetic_packed", "dataset_format": "synthetic", "packing": True, "packing_strategy": "first_fit",
            "packing_length": 256, "extra_kwargs": {"vocab_size": vocab, "min_len": 16, "max_len": 128}}


def _vision(media: str = "image") -> dict:
    return {"dataset_type": "synthetic_vl", "dataset_format": "synthetic", "packing": True, "packing_length": 256,
            "extra_kwargs": {"vocab_size": 500, "media": media, "num_media": [1, 2], "size": [32, 64], "size_multiple": 16, "frames": [2, 4],
                             "patch_size": 8, "temporal_patch_size": 2, "merge_size": 2, "image_token_id": 501, "video_token_id": 502,
                             "pixel_dtype": "float32"}}


def _tensors(spec: dict) -> dict:
    return {"dataset_type": "synthetic_tensors", "dataset_format": "synthetic", "extra_kwargs": {"spec": spec}}


def _vl(model_type: str, text: dict) -> dict:
    return dict(model_type=model_type, text_config=dict(text), vision_config=dict(VISION), image_token_id=501, video_token_id=502,
                vision_start_token_id=503)


# family -> (model_type, model config, dataset, extra trainer arguments)
FAMILIES: Dict[str, tuple] = {
    "qwen2_5": ("qwen2", LM, _packed(), {}),
    "qwen3": ("qwen3", LM, _packed(), {"use_muon": True}),
    "qwen3_sp": ("qwen3", LM, _packed(), {"sp_ulysses_degree": 2}),
    "qwen3_moe": ("qwen3_moe", MOE, _packed(), {}),
    "qwen3_moe_ep": ("qwen3_moe", MOE, _packed(), {"ep_degree": 2}),
    "qwen3_5": ("qwen3_5_text", HYBRID, _packed(), {}),
    "qwen3_5_moe": ("qwen3_5_moe_text", dict(HYBRID, **{k: MOE[k] for k in ("num_experts", "num_experts_per_tok", "moe_intermediate_size",
                                                                          "norm_topk_prob", "router_aux_loss_coef")}), _packed(), {}),
    "qwen3_vl": ("qwen3_vl", _vl("qwen3_vl", VL_TEXT), _vision("image"), {}),
    "qwen3_vl_video": ("qwen3_vl", _vl("qwen3_vl", VL_TEXT), _vision("video"), {}),
    "qwen3_vl_moe": ("qwen3_vl_moe", _vl("qwen3_vl_moe", dict(VL_TEXT, **{k: MOE[k] for k in ("num_experts", "num_experts_per_tok",
                                                                                           "moe_intermediate_size", "norm_topk_prob")})),
                     _vision("image"), {}),
    "qwen3_tp": ("qwen3", LM, _packed(), {"tp_degree": 2}),
    "qwen3_vl_sp": ("qwen3_vl", _vl("qwen3_vl", VL_TEXT), _vision("video"), {"sp_ulysses_degree": 2}),
    "qwen3_vl_tp": ("qwen3_vl", _vl("qwen3_vl", VL_TEXT), _vision("image"), {"tp_degree": 2}),
    "qwen3_vl_moe_ep": ("qwen3_vl_moe", _vl("qwen3_vl_moe", dict(VL_TEXT, **{k: MOE[k] for k in ("num_experts", "num_experts_per_tok",
                                                                                              "moe_intermediate_size", "norm_topk_prob")})),
                        _vision("image"), {"ep_degree": 2}),
    "qwen3_5_moe_ep": ("qwen3_5_moe_text", dict(HYBRID, **{k: MOE[k] for k in ("num_experts", "num_experts_per_tok", "moe_intermediate_size",
                                                                             "norm_topk_prob", "router_aux_loss_coef")}), _packed(),
                       {"ep_degree": 2}),
    "qwen3_5_sp": ("qwen3_5_text", HYBRID, _packed(), {"sp_ulysses_degree": 2}),
    "qwen2_5_vl": ("qwen2_5_vl", dict(model_type="qwen2_5_vl", text_config=dict(LM, rope_scaling={"mrope_section": [8, 4, 4]}),
                                      vision_config=dict(depth=2, hidden_size=128, intermediate_size=256, num_heads=4, patch_size=8,
                                                         temporal_patch_size=2, spatial_merge_size=2, out_hidden_size=128, window_size=32,
                                                         fullatt_block_indexes=[1], in_channels=3),
                                      image_token_id=501, video_token_id=502, vision_start_token_id=503), _vision("image"), {}),
    "llavaonevision1_5": ("llavaonevision1_5", dict(model_type="llavaonevision1_5", text_config=dict(LM, rope_theta=10000.0),
                                                    vision_config=dict(depth=2, hidden_size=128, intermediate_size=256, num_heads=4, patch_size=8,
                                                                       spatial_merge_size=2, text_hidden_size=128, hidden_act="gelu",
                                                                       layer_norm_eps=1e-5),
                                                    image_token_id=501, video_token_id=502),
                          _vision("image") | {"extra_kwargs": dict(_vision("image")["extra_kwargs"], temporal_patch_size=1)}, {}),
    "qwen3_dllm": ("qwen3_dllm", dict(LM, mask_token_id=511), _packed() | {"extra_kwargs": {"vocab_size": 500, "min_len": 16, "max_len": 128,
                                                                                           "collator_type": "dllm", "mask_token_id": 511}},
                   {"trainer_type": "dllm_trainer"}),
    "hf_trainer": ("qwen2", LM, _packed(), {"trainer_type": "hf_trainer", "average_tokens_across_devices": True}),
    "grpo": ("qwen2", LM, _packed() | {"extra_kwargs": {"vocab_size": 512, "min_len": 16, "max_len": 64, "prompt_len": 4}},
             {"trainer_type": "grpo_trainer", "rl_config": {"group_size": 4, "max_new_tokens": 6, "reward": "repeat_last_prompt_token", "beta": 0.01}}),
    "sit": ("sit", dict(input_size=8, hidden_size=128, depth=2, num_heads=4, num_classes=10),
            _tensors({"pixel_values": {"shape": [4, 8, 8]}, "labels": {"shape": [], "kind": "randint", "high": 10}}),
            {"trainer_type": "sit_trainer", "per_device_train_batch_size": 2}),
    "wanvideo": ("wanvideo", dict(dim=128, ffn_dim=256, num_heads=4, num_layers=2, text_dim=64, in_dim=4, out_dim=4),
                 _tensors({"latents": {"shape": [4, 2, 8, 8]}, "context": {"shape": [5, 64]}}),
                 {"trainer_type": "wan_trainer", "per_device_train_batch_size": 2}),
    "rae_siglip": ("rae_siglip", dict(image_size=32, patch_size=8, encoder_dim=128, encoder_depth=1, encoder_heads=2, decoder_dim=128,
                                      decoder_depth=1, decoder_heads=2), _tensors({"pixel_values": {"shape": [3, 32, 32]}}),
                   {"trainer_type": "rae_trainer", "per_device_train_batch_size": 2,
                    "gan_config": dict(discriminator="patch", disc_dim=32, perceptual_weight=0.0, discriminator_start_step=0,
                                       discriminator_loss_start_step=0)}),
}


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def write_config(name: str, out: str, steps: int, cpu: bool) -> str:
    import yaml

    model_type, model_cfg, dataset, extra = FAMILIES[name]
    extra = dict(extra)
    trainer_type = extra.pop("trainer_type", "fsdp2_trainer")
    targs = dict(output_dir=out, max_steps=steps, learning_rate=1e-3, per_device_train_batch_size=1, logging_steps=1, save_strategy="no",
                 lr_scheduler_type="constant", seed=0, use_cpu=cpu, bf16=not cpu, ddp_timeout=120, report_to="none")
    targs.update(extra)
    cfg = [{"type": "trainer", "config": {"trainer_type": trainer_type, "dataset_config": dataset,
                                          "model_config": {"load_from_config": {"model_type": model_type, "config": model_cfg}},
                                          "trainer_args": targs}}]
    path = os.path.join(out, f"{name}.yaml")
    with open(path, "w") as f:
        yaml.safe_dump(cfg, f)
    return path


def run_family(name: str, ranks: int, steps: int, cpu: bool, timeout: int, verbose: bool) -> Optional[str]:
    """``None`` when the family trained; otherwise one line saying what went wrong."""
    with tempfile.TemporaryDirectory(prefix=f"train_suite_{name}_") as out:
        cfg = write_config(name, out, steps, cpu)
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={ranks}", "--master-addr", "127.0.0.1",
               "--master-port", str(free_port()), "-m", "lmms_engine_b200.launch.cli", f"config_yaml={cfg}"]
        env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""), OMP_NUM_THREADS="2")
        if not cpu:
            env.setdefault("CUDA_VISIBLE_DEVICES", ",".join(str(i) for i in range(ranks)))
        t0 = time.time()
        try:
            proc = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=timeout)
        except subprocess.TimeoutExpired:
            return f"no exit within {timeout} s"
        log = proc.stdout + proc.stderr
        if verbose or proc.returncode != 0:
            print(log[-4000:])
        if proc.returncode != 0:
            return f"exit code {proc.returncode}"
        losses = [float(x) for x in re.findall(r"train/loss=([^\s,]+)", log)]
        if len(losses) < steps or not all(math.isfinite(x) for x in losses):
            return f"expected {steps} finite losses in the log, found {losses}"
        print(f"  {name}: ok in {time.time() - t0:.0f} s")
        return None


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model-name", default="", help="families of the table separated by commas, or a prefix of several (default: all)")
    ap.add_argument("--gpu-count", type=int, default=2, help="ranks per run (GPUs, or CPU processes with --cpu)")
    ap.add_argument("--cpu", action="store_true", help="gloo ranks on the CPU in fp32")
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--timeout", type=int, default=600)
    ap.add_argument("--no-verbose", action="store_true")
    ap.add_argument("--list", action="store_true")
    a = ap.parse_args(argv)
    wanted = [w for w in a.model_name.split(",") if w] or [""]
    names = [n for n in FAMILIES if any(n == w for w in wanted)] or [n for n in FAMILIES if any(n.startswith(w) for w in wanted)]
    if a.list:
        print("\n".join(names))
        return 0
    if not names:
        print(f"no family matches {a.model_name!r}; known: {', '.join(FAMILIES)}")
        return 2
    failed = {}
    for name in names:
        need = max(int(FAMILIES[name][3].get(k, 1)) for k in ("sp_ulysses_degree", "ep_degree", "tp_degree"))
        if a.gpu_count % need:
            print(f"  {name}: skipped (needs a multiple of {need} ranks)")
            continue
        why = run_family(name, a.gpu_count, a.steps, a.cpu, a.timeout, not a.no_verbose)
        if why:
            failed[name] = why
            print(f"  {name}: FAILED ({why})")
    print(json.dumps({"ran": len(names), "failed": failed}))
    return 1 if failed else 0


if __name__ == "__main__":
    sys.exit(main())
