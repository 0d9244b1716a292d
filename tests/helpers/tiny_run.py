"""Runs the tiny Qwen2.5-style plumbing configuration through ``create_train_task`` and
writes the per-step losses to a JSON file (rank 0).  Launched by the CPU tests, alone or
under ``torch.distributed.run`` with the gloo backend."""
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


MOE = dict(vocab_size=4096, hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
           head_dim=32, rms_norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=False, num_experts=4, num_experts_per_tok=2,
           moe_intermediate_size=64, norm_topk_prob=True, router_aux_loss_coef=0.001)


def make_config(out, runtime="auto", steps=10, pattern="uniform", extra_args=None, sp=1, data_extra=None, model="dense"):
    targs = dict(output_dir=out, max_steps=steps, learning_rate=1e-3, per_device_train_batch_size=1, use_cpu=True,
                 bf16=False, logging_steps=1, save_strategy="no", lr_scheduler_type="constant", sharding_runtime=runtime,
                 seed=1, adam_beta2=0.95, sp_ulysses_degree=sp)
    targs.update(extra_args or {})
    return {
        "trainer_type": "fsdp2_trainer",
        "dataset_config": {
            "dataset_type": "synthetic_packed", "dataset_format": "synthetic", "packing": True,
            "packing_strategy": "first_fit", "packing_length": 1024, "data_seed": 7,
            "extra_kwargs": {"vocab_size": 4096, "min_len": 32, "max_len": 512, "pattern": pattern, **(data_extra or {})},
        },
        "model_config": {"load_from_config": {"model_type": "qwen2", "config": dict(
            vocab_size=4096, hidden_size=256, intermediate_size=688, num_hidden_layers=4, num_attention_heads=4,
            num_key_value_heads=2, head_dim=64, rms_norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=True)}},
        "trainer_args": targs,
    } if model == "dense" else {
        "trainer_type": "fsdp2_trainer",
        "dataset_config": {
            "dataset_type": "synthetic_packed", "dataset_format": "synthetic", "packing": True,
            "packing_strategy": "first_fit", "packing_length": 512, "data_seed": 7,
            "extra_kwargs": {"vocab_size": 4096, "min_len": 32, "max_len": 256, "pattern": pattern, **(data_extra or {})},
        },
        "model_config": {"load_from_config": {"model_type": "qwen3_moe", "config": dict(MOE)}},
        "trainer_args": targs,
    }


def main():
    import argparse

    ap = argparse.ArgumentParser()
    ap.add_argument("--out", required=True)
    ap.add_argument("--runtime", default="auto")
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--pattern", default="uniform")
    ap.add_argument("--sp", type=int, default=1)
    ap.add_argument("--extra", default="{}")
    ap.add_argument("--data_extra", default="{}")
    ap.add_argument("--model", default="dense", choices=["dense", "moe"])
    a = ap.parse_args()
    from lmms_engine_b200.launch.cli import create_train_task

    runner = create_train_task(make_config(a.out, a.runtime, a.steps, a.pattern, json.loads(a.extra), a.sp, json.loads(a.data_extra), a.model)).build()
    hist = runner.run()
    if int(os.environ.get("RANK", "0")) == 0:
        with open(os.path.join(a.out, "losses.json"), "w") as f:
            json.dump({"loss": [h["train/loss"] for h in hist], "grad_norm": [h["train/grad_norm"] for h in hist],
                       "final_step": runner.trainer.global_step}, f)
    import torch.distributed as dist

    if dist.is_initialized():
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
