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


@pytest.mark.parametrize("family", ["qwen3", "qwen3_moe", "qwen3_5_text"])
def test_generation_on_cached_keys_matches_rerunning_the_sequences(family):
    """Prefill + one token per step against the key / value cache gives the hidden states of the full pass and the
    same sampled completions (EOS at different steps, a rank kept running by its group)."""
    from lmms_engine_b200.mapping_func import create_model_from_config
    from lmms_engine_b200.models.kv_cache import PackedKVCache
    from lmms_engine_b200.train.rl.grpo_trainer import sample_completions

    torch.manual_seed(0)
    cfg = dict(vocab_size=64, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
               head_dim=8, max_position_embeddings=128)
    if family == "qwen3_moe":
        cfg.update(num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32, norm_topk_prob=True)
    if family == "qwen3_5_text":  # hybrid: linear-attention layers keep a convolution tail and a state matrix per sequence
        cfg.update(num_hidden_layers=4, linear_conv_kernel_dim=4, linear_key_head_dim=8, linear_value_head_dim=8, linear_num_key_heads=2,
                   linear_num_value_heads=4, rope_parameters={"rope_theta": 10000.0, "partial_rotary_factor": 0.5})
    model = create_model_from_config(family, dict(cfg, model_type=family)).eval()
    seqs = [torch.randint(0, 64, (n,)) for n in (9, 5, 12)]
    with torch.no_grad():
        cu = torch.tensor([0, 9, 14, 26], dtype=torch.int32)
        full = model(input_ids=torch.cat(seqs), cu_seqlens=cu)["hidden_states"]
        cache = PackedKVCache(cfg["num_hidden_layers"], [16, 16, 16])
        heads = [6, 5, 7]  # prefill lengths; the rest arrives in two uneven passes, the second sequence sits one out
        pos = cache.advance(heads)
        ids = torch.cat([s[:h] for s, h in zip(seqs, heads)])
        first = model(input_ids=ids, cu_seqlens=torch.tensor([0, 6, 11, 18], dtype=torch.int32), position_ids=pos, kv_cache=cache)["hidden_states"]
        pos = cache.advance([3, 0, 2])
        assert pos.tolist() == [6, 7, 8, 7, 8]
        second = model(input_ids=torch.cat([seqs[0][6:9], seqs[2][7:9]]), cu_seqlens=torch.tensor([0, 3, 5], dtype=torch.int32),
                       position_ids=pos, kv_cache=cache)["hidden_states"]
        pos = cache.advance([0, 0, 3])
        third = model(input_ids=seqs[2][9:], cu_seqlens=torch.tensor([0, 3], dtype=torch.int32), position_ids=pos, kv_cache=cache)["hidden_states"]
    pieces = torch.cat([first[:6], second[:3], first[6:11], first[11:18], second[3:5], third])
    assert torch.allclose(pieces, full, atol=2e-5), float((pieces - full).abs().max())
    with pytest.raises(ValueError):
        cache.advance([8, 0, 0])  # 9 held + 8 > 16
    prompts = [torch.randint(0, 64, (n,)) for n in (4, 7, 3)]
    runs = [sample_completions(model, prompts, 12, 1.0, eos_token_id=5, generator=torch.Generator().manual_seed(11), use_cache=flag)
            for flag in (True, False)]
    assert all(torch.equal(a, b) for a, b in zip(*runs)) and any(r.numel() < 12 for r in runs[0])
    assert model.supports_kv_cache


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
