"""Every registered trainer runs a few steps end to end on CPU through ``create_train_task``
with a tiny native model and synthetic data."""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

TINY_LM = dict(vocab_size=128, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
               num_key_value_heads=2, head_dim=16)


def _run(tmp_path, trainer_type, model_type, model_cfg, dataset, steps=3, **targs):
    import torch.distributed as dist

    from lmms_engine_b200.launch.cli import create_train_task

    os.environ.setdefault("MASTER_PORT", "29731")
    cfg = {
        "trainer_type": trainer_type,
        "dataset_config": dataset,
        "model_config": {"load_from_config": {"model_type": model_type, "config": model_cfg}},
        "trainer_args": dict(output_dir=str(tmp_path), max_steps=steps, learning_rate=1e-3, use_cpu=True, bf16=False,
                             logging_steps=1, save_strategy="no", lr_scheduler_type="constant", seed=0, **targs),
    }
    runner = create_train_task(cfg).build()
    hist = runner.run()
    assert len(hist) == steps and all(h["train/loss"] == h["train/loss"] for h in hist)
    return hist, runner


def _packed(**extra):
    return {"dataset_type": "synthetic_packed", "dataset_format": "synthetic", "packing": True, "packing_length": 256,
            "extra_kwargs": {"vocab_size": 120, "min_len": 16, "max_len": 64, "pattern": "periodic", **extra}}


def _tensors(spec):
    return {"dataset_type": "synthetic_tensors", "dataset_format": "synthetic", "extra_kwargs": {"spec": spec}}


def test_hf_trainer_token_weighted_loss(tmp_path):
    hist, _ = _run(tmp_path, "hf_trainer", "qwen2", TINY_LM, _packed(), average_tokens_across_devices=True)
    assert hist[-1]["train/loss"] < hist[0]["train/loss"] + 0.5


def test_dllm_trainer_logs_nll(tmp_path):
    hist, _ = _run(tmp_path, "dllm_trainer", "qwen3_dllm", dict(TINY_LM, mask_token_id=127),
                   _packed(collator_type="dllm", mask_token_id=127))
    assert "train/nll" in hist[0]


def test_sit_trainer_keeps_ema_copy(tmp_path):
    spec = {"pixel_values": {"shape": [4, 8, 8]}, "labels": {"shape": [], "kind": "randint", "high": 10}}
    _, runner = _run(tmp_path, "sit_trainer", "sit", dict(input_size=8, hidden_size=64, depth=2, num_heads=4, num_classes=10),
                     _tensors(spec), per_device_train_batch_size=2)
    assert runner.trainer.ema_model is not None


def test_wan_trainer_flow_matching(tmp_path):
    spec = {"latents": {"shape": [4, 2, 8, 8]}, "context": {"shape": [5, 32]}}
    _run(tmp_path, "wan_trainer", "wanvideo", dict(dim=64, ffn_dim=128, num_heads=4, num_layers=2, text_dim=32, in_dim=4, out_dim=4),
         _tensors(spec), per_device_train_batch_size=2)


def test_rae_trainer_gan_steps(tmp_path):
    spec = {"pixel_values": {"shape": [3, 32, 32]}}
    _, runner = _run(tmp_path, "rae_trainer", "rae_siglip",
                     dict(image_size=32, patch_size=8, encoder_dim=32, encoder_depth=1, encoder_heads=2, decoder_dim=32,
                          decoder_depth=1, decoder_heads=2), _tensors(spec), per_device_train_batch_size=2,
                     gan_config=dict(discriminator="patch", disc_dim=32, perceptual_weight=0.0, discriminator_start_step=0,
                                     discriminator_loss_start_step=0))
    assert runner.trainer.ema_state and runner.trainer.loss_parts["disc_loss"] > 0


def test_grpo_trainer_improves_reward_signal(tmp_path):
    hist, runner = _run(tmp_path, "grpo_trainer", "qwen2", TINY_LM, _packed(prompt_len=4), steps=2,
                        rl_config={"group_size": 4, "max_new_tokens": 6, "reward": "repeat_last_prompt_token", "beta": 0.01})
    assert "rl/reward_mean" in hist[0] and "rl/kl" in hist[0]


def test_grpo_trainer_steps_once_per_accumulation_window(tmp_path):
    """With gradient accumulation the optimizer moves once per window, together with global_step."""
    hist, runner = _run(tmp_path, "grpo_trainer", "qwen2", TINY_LM, _packed(prompt_len=4), steps=2, gradient_accumulation_steps=2,
                        rl_config={"group_size": 2, "max_new_tokens": 4, "reward": "length", "beta": 0.0})
    assert runner.trainer.runtime.step_count == 2
    with pytest.raises(ValueError, match="num_iterations"):
        _run(tmp_path, "grpo_trainer", "qwen2", TINY_LM, _packed(prompt_len=4), steps=1, gradient_accumulation_steps=2,
             rl_config={"group_size": 2, "max_new_tokens": 2, "num_iterations": 2})


def test_grpo_math():
    from lmms_engine_b200.train.rl import group_advantages, grpo_token_loss

    adv = group_advantages(torch.tensor([1.0, 0.0, 0.0, 1.0, 2.0, 2.0, 2.0, 2.0]), 4)
    assert torch.allclose(adv[:4], torch.tensor([1.0, -1.0, -1.0, 1.0]), atol=1e-3) and adv[4:].abs().max() < 1e-3
    logp = torch.tensor([-1.0, -2.0], requires_grad=True)
    loss, kl = grpo_token_loss(logp, logp.detach(), logp.detach(), torch.tensor([1.0, -1.0]), torch.ones(2), 0.2, 0.1)
    loss.backward()
    assert torch.allclose(logp.grad, torch.tensor([-0.5, 0.5])) and float(kl) == 0.0


def test_transformers_fallback_family_trains(tmp_path):
    """A model family without a native implementation is built from the transformers library and
    trained by the same trainer on padded batches."""
    pytest.importorskip("transformers")
    cfg = dict(vocab_size=128, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
               num_key_value_heads=2, max_position_embeddings=256)
    hist, runner = _run(tmp_path, "fsdp2_trainer", "mistral", cfg, _packed(collator_type="padded"), steps=4)
    assert type(runner.model).__module__.startswith("transformers")
    assert hist[-1]["train/loss"] < hist[0]["train/loss"] + 0.5


def test_flow_grpo_trainer_samples_scores_and_replays_image_generation(tmp_path):
    """Unified model: groups of images sampled per prompt with recorded SDE steps, rewards normalised per group, the
    policy replays every recorded step and the optimizer moves after each."""
    cfg = dict(model_type="bagel", vocab_size=128, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
               num_key_value_heads=2, head_dim=8, latent_channels=4, latent_patch_size=2, max_latent_size=8, layer_module="Qwen2MoTDecoderLayer")
    hist, runner = _run(tmp_path, "flow_grpo_trainer", "bagel", cfg, _packed(prompt_len=4), steps=2,
                        rl_config={"group_size": 3, "image_hw": [2, 2], "num_timesteps": 5, "sde_window": [1, 2], "noise_level": 0.7,
                                   "reward": "latent_brightness", "boi_token_id": 126, "eoi_token_id": 127, "beta": 0.01, "clip_range": [1e-3, 1e-3]})
    assert "rl/reward_mean" in hist[0] and hist[0]["rl/recorded_steps"] > 0 and "rl/policy_loss" in hist[0]
    assert runner.trainer.ref_model is not None
