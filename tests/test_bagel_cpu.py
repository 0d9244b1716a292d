"""Bagel: per-split attention rules on the varlen kernel against the dense mask, full mixture-of-transformers layers,
understanding tokens from the packed SigLIP tower, in-model autoencoder, rollout and policy-gradient pass."""
import math
import os
import sys

import pytest
import torch
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

BASE = dict(model_type="bagel", vocab_size=120, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
            num_key_value_heads=2, head_dim=8, latent_channels=4, latent_patch_size=2, max_latent_size=8, attention_bias=True)


def _dense_mask(sample_lens, split_lens, modes):
    """The rules stated directly: one boolean [T, T] mask over the packed stream."""
    T = sum(sample_lens)
    mask = torch.zeros(T, T, dtype=torch.bool)
    tok, si = 0, 0
    for n in sample_lens:
        start, end = tok, tok + n
        spans = []
        while tok < end:
            spans.append((tok, tok + split_lens[si], modes[si]))
            tok += split_lens[si]
            si += 1
        for a, b, m in spans:
            mask[a:b, start:a] = True
            mask[a:b, a:b] = torch.ones(b - a, b - a).tril().bool() if m == "causal" else True
        for a, b, m in spans:
            if m == "noise":
                mask[:, a:b] = False
                mask[a:b, a:b] = True
    return mask


def test_split_plan_reproduces_the_dense_mask():
    from lmms_engine_b200.models.bagel import build_split_plan, split_attention
    from lmms_engine_b200.models.decoder_lm import PackedContext

    torch.manual_seed(0)
    sample_lens, split_lens = [17, 9], [5, 6, 2, 4, 3, 6]
    modes = ["causal", "noise", "causal", "full", "causal", "noise"]
    T = sum(sample_lens)
    q, k, v = torch.randn(T, 4, 8), torch.randn(T, 2, 8), torch.randn(T, 2, 8)
    ctx = PackedContext(torch.tensor([0, 17, 26], dtype=torch.int32), 26, None, None, True)
    ctx.split_plan = build_split_plan(sample_lens, split_lens, modes, q.device)
    got = split_attention(q, k, v, ctx, 1 / math.sqrt(8))
    mask = _dense_mask(sample_lens, split_lens, modes)
    kk, vv = k.repeat_interleave(2, 1), v.repeat_interleave(2, 1)
    want = F.scaled_dot_product_attention(q.transpose(0, 1), kk.transpose(0, 1), vv.transpose(0, 1), attn_mask=mask).transpose(0, 1)
    assert (got - want).abs().max() < 1e-5
    # a later token never sees a noised image; the noised image sees what came before it
    assert not mask[11, 5:11].any() and mask[11, :5].all() and mask[7, :5].all() and mask[7, 5:11].all() and not mask[14, 5:11].any()
    with pytest.raises(ValueError):
        build_split_plan([10], [4, 4], ["causal", "full"], q.device)


def test_full_mixture_of_transformers_layers_and_checkpoint_names():
    from lmms_engine_b200.mapping_func import create_model_from_config

    torch.manual_seed(0)
    model = create_model_from_config("bagel", dict(BASE, layer_module="Qwen2MoTDecoderLayer", qk_norm=True))
    names = set(model.state_dict())
    for k in ("model.layers.0.self_attn.q_proj_moe_gen.weight", "model.layers.0.self_attn.o_proj_moe_gen.weight",
              "model.layers.0.self_attn.k_norm_moe_gen.weight", "model.layers.1.input_layernorm_moe_gen.weight",
              "model.layers.1.post_attention_layernorm_moe_gen.weight", "model.layers.1.mlp_moe_gen.down_proj.weight", "model.norm_moe_gen.weight",
              "time_embedder.mlp.0.weight", "latent_pos_embed.pos_embed", "vae2llm.weight", "llm2vae.bias"):
        assert k in names, k
    conv = model.convert_hf_state_dict({"language_model.model.norm_moe_gen.weight": torch.ones(32), "vae2llm.bias": torch.zeros(32)})
    assert set(conv) == {"model.norm_moe_gen.weight", "vae2llm.bias"}
    ids = torch.randint(0, 100, (30,))
    lat_idx = torch.arange(10, 16)
    batch = dict(input_ids=ids, labels=ids, cu_seqlens=torch.tensor([0, 30], dtype=torch.int32), latent_tokens=torch.randn(6, 16),
                 latent_index=lat_idx, latent_pos=torch.tensor([0, 1, 2, 8, 9, 10]), timesteps=torch.full((6,), 0.6),
                 split_lens=[10, 6, 14], attn_modes=["causal", "noise", "causal"])
    out = model(**batch)
    out["loss"].backward()
    # generation tokens trained their own projections, norms and MLP; understanding tokens theirs
    layer = model.model.layers[0]
    for p in (layer.self_attn.q_proj_moe_gen.weight, layer.self_attn.o_proj_moe_gen.weight, layer.mlp_moe_gen.gate_proj.weight,
              layer.input_layernorm_moe_gen.weight, layer.self_attn.q_proj.weight, layer.mlp.gate_proj.weight, model.model.norm_moe_gen.weight):
        assert p.grad is not None and p.grad.abs().sum() > 0
    # swapping the two parameter sets changes the result: the routing by token type is real
    with torch.no_grad():
        a = model(**dict(batch, noise=torch.zeros(6, 16)))["velocity"]
        w = layer.mlp_moe_gen.gate_proj.weight
        w.add_(0.5)
        b = model(**dict(batch, noise=torch.zeros(6, 16)))["velocity"]
    assert (a - b).abs().max() > 1e-4
    # text after a noised image does not depend on it ("noise" splits are invisible to the rest)
    with torch.no_grad():
        model.eval()
        h1 = model(**dict(batch, noise=torch.zeros(6, 16), labels=None))
        lat2 = batch["latent_tokens"] + 3.0
        e1, *_ = model.embed_stream(ids, batch["latent_tokens"], lat_idx, batch["latent_pos"], batch["timesteps"], noise=torch.zeros(6, 16))
        e2, *_ = model.embed_stream(ids, lat2, lat_idx, batch["latent_pos"], batch["timesteps"], noise=torch.zeros(6, 16))
        pos, cu = torch.arange(30), batch["cu_seqlens"]
        o1 = model.run_decoder(e1, pos, cu, lat_idx, batch["split_lens"], batch["attn_modes"])
        o2 = model.run_decoder(e2, pos, cu, lat_idx, batch["split_lens"], batch["attn_modes"])
    assert (o1[16:] - o2[16:]).abs().max() < 1e-5 and (o1[10:16] - o2[10:16]).abs().max() > 1e-3


def test_understanding_images_and_in_model_autoencoder():
    from lmms_engine_b200.mapping_func import create_model_from_config
    from lmms_engine_b200.models.bagel_parts import flattened_position_ids, patchify_image

    torch.manual_seed(0)
    vit = dict(hidden_size=32, intermediate_size=64, num_hidden_layers=3, num_attention_heads=4, image_size=32, patch_size=8)
    vae = dict(resolution=32, ch=32, ch_mult=[1, 2, 4, 4], num_res_blocks=1, downsample=8)
    model = create_model_from_config("bagel", dict(BASE, visual_und=True, vit_config=vit, vit_rope=True, vit_select_layer=-2,
                                                   vit_max_num_patch_per_side=4, vae_config=vae))
    assert len(model.vit_model.vision_model.encoder.layers) == 2  # the last block is not used
    assert not any(p.requires_grad for p in model.vae_model.parameters())
    model.train()
    assert not model.vae_model.training
    img_u = torch.randn(3, 16, 32)  # understanding image: 2 x 4 patches
    vit_tokens = patchify_image(img_u, 8)
    vit_pos = flattened_position_ids(16, 32, 8, 4)
    assert vit_pos.tolist() == [0, 1, 2, 3, 4, 5, 6, 7]
    assert flattened_position_ids(16, 16, 8, 4, interpolate=True).tolist() == [0, 2, 8, 10]
    gen = torch.randn(1, 3, 32, 48) .clamp(-1, 1)  # generation target: latent 4 x 6 -> 2 x 3 patches
    ids = torch.randint(0, 100, (30,))
    batch = dict(input_ids=ids, labels=ids, cu_seqlens=torch.tensor([0, 30], dtype=torch.int32), vit_tokens=vit_tokens,
                 vit_index=torch.arange(2, 10), vit_position_ids=vit_pos, vit_seqlens=torch.tensor([8]), images=gen, latent_shapes=[(2, 3)],
                 latent_index=torch.arange(20, 26), latent_pos=torch.tensor([0, 1, 2, 8, 9, 10]), timesteps=torch.full((6,), 0.4),
                 split_lens=[2, 8, 10, 6, 4], attn_modes=["causal", "full", "causal", "noise", "causal"])
    out = model(**batch)
    assert out["velocity"].shape == (6, 16) and torch.isfinite(out["loss"])
    out["loss"].backward()
    assert model.connector.fc1.weight.grad.abs().sum() > 0 and model.vit_model.vision_model.encoder.layers[0].mlp.fc1.weight.grad.abs().sum() > 0
    # the latents the model made are the autoencoder's, patch by patch
    lat = model.latents_from_images(gen, [(2, 3)])
    z = model.vae_model.encode(gen)  # sampling posterior: compare shapes and the deterministic part
    assert lat.shape == (6, 16) and z.shape == (1, 4, 4, 6)
    model.vae_model.sample = False
    lat = model.latents_from_images(gen, [(2, 3)])
    z = model.vae_model.encode(gen)[0]
    assert torch.allclose(lat[1].view(2, 2, 4), z[:, 0:2, 2:4].permute(1, 2, 0), atol=1e-6)
    assert torch.allclose(model.unpatchify_latent(lat, (2, 3)), z, atol=1e-6)


def test_rollout_records_steps_and_the_policy_pass_reproduces_their_log_probabilities():
    from lmms_engine_b200.mapping_func import create_model_from_config

    torch.manual_seed(0)
    model = create_model_from_config("bagel", dict(BASE, layer_module="Qwen2MoTDecoderLayer")).eval()
    with torch.no_grad():
        model.llm2vae.weight.normal_(0, 0.05)
    prompt, uncond = torch.randint(0, 100, (7,)), torch.randint(0, 100, (2,))
    g = torch.Generator().manual_seed(3)
    roll = model.generate_image(prompt, (2, 3), boi_id=101, eoi_id=102, num_timesteps=6, noise_level=0.7, sde_window=(1, 3), uncond_ids=uncond,
                                cfg_text_scale=2.0, generator=g)
    assert len(roll["latents"]) == 3 and roll["image_latent"].shape == (6, 16)
    assert roll["timesteps"] == sorted(roll["timesteps"], reverse=True) and all(a > b for a, b in zip(roll["timesteps"], roll["next_timesteps"]))
    assert roll["stream"]["split_lens"] == [7, 8] and roll["stream"]["pos"][7:].tolist() == [7] * 8
    # the same policy assigns the recorded steps the recorded log-probabilities: ratio 1, loss = -advantage
    stats = model.grpo_learn(roll, advantage=0.8, clip_range=(1e-4, 1e-4), cfg_text_scale=2.0)
    assert abs(float(stats["policy_loss"]) + 0.8) < 1e-4 and float(stats["clipfrac"]) == 0.0
    # gradients flow through the step mean, one backward per recorded step
    model.train()
    seen = []
    model.grpo_learn(roll, advantage=-1.0, cfg_text_scale=2.0, step_callback=lambda loss: (loss.backward(), seen.append(float(loss))))
    assert len(seen) == 3 and model.llm2vae.weight.grad.abs().sum() > 0
    # KL to a reference policy: zero against itself, positive against a perturbed copy
    import copy

    ref = copy.deepcopy(model).eval()
    model.eval()
    same = model.grpo_learn(roll, advantage=0.5, beta=0.1, ref_model=ref, cfg_text_scale=2.0)
    assert float(same["kl_loss"]) < 1e-10
    with torch.no_grad():
        ref.llm2vae.bias.add_(0.3)
    other = model.grpo_learn(roll, advantage=0.5, beta=0.1, ref_model=ref, cfg_text_scale=2.0)
    assert float(other["kl_loss"]) > 1e-4
    # without noise the sampler is the deterministic Euler solver and records nothing
    det = model.generate_image(prompt, (2, 3), boi_id=101, eoi_id=102, num_timesteps=4, noise_level=0.0)
    assert det["latents"] == [] and torch.isfinite(det["image_latent"]).all()


@pytest.mark.parametrize("layer_module", ["Qwen2DecoderLayer", "Qwen2MoEDecoderLayer", "Qwen2MoTDecoderLayer"])
def test_sampling_on_recorded_prompt_keys_equals_the_full_stream(layer_module):
    """Running the prompt once and every step on the image block against its keys / values gives the image of the
    full-stream sampler, with and without guidance; the record handed to the learning pass stays complete."""
    from lmms_engine_b200.mapping_func import create_model_from_config

    torch.manual_seed(1)
    model = create_model_from_config("bagel", dict(BASE, layer_module=layer_module)).eval()
    with torch.no_grad():
        model.llm2vae.weight.normal_(0, 0.05)
    prompt, uncond = torch.randint(0, 100, (9,)), torch.randint(0, 100, (3,))
    for kw in (dict(), dict(uncond_ids=uncond, cfg_text_scale=3.0)):
        runs = [model.generate_image(prompt, (3, 2), boi_id=101, eoi_id=102, num_timesteps=5, noise_level=0.5, use_cache=flag,
                                     generator=torch.Generator().manual_seed(7), **kw) for flag in (True, False)]
        assert torch.allclose(runs[0]["image_latent"], runs[1]["image_latent"], atol=2e-5)
        assert torch.allclose(torch.stack(runs[0]["log_probs"]), torch.stack(runs[1]["log_probs"]), atol=1e-3)
        assert set(runs[0]["stream"]) == set(runs[1]["stream"]) and "prefix" not in runs[0]["stream"]
    cached = model.cache_prompt(model.image_stream(prompt, (3, 2), 101, 102))
    assert len(cached["prefix"]) == 2 and cached["prefix"][0][0].shape == (9, 2, 8) and cached["block"]["ids"].numel() == 8
    bare = model.image_stream(prompt[:0], (3, 2), 101, 102)
    assert model.cache_prompt(bare) is bare  # nothing in front of the image: nothing to record


def test_taylor_forecaster_schedule_and_expansion():
    """Computed steps: the first ``first_enhance``, then every ``interval``-th; a quadratic in the step index is forecast
    exactly once two derivatives exist; sampling with forecasts runs the decoder less often and stays close."""
    from lmms_engine_b200.mapping_func import create_model_from_config
    from lmms_engine_b200.models.bagel import TaylorForecaster

    fc = TaylorForecaster(interval=3, max_order=2, first_enhance=5)
    f = lambda s: torch.tensor([1.0 + 0.5 * s + 0.25 * s * s, -2.0 * s])  # noqa: E731
    ran, worst = [], 0.0
    for step in range(14):
        if fc.wants_model(step):
            fc.update(step, f(step))
            ran.append(step)
        elif len(fc.factors) == 3 and step > 9:
            worst = max(worst, float((fc.forecast(step) - f(step)).abs().max()))
    assert ran == [0, 1, 2, 3, 4, 7, 10, 13]
    # backward differences of a quadratic over uneven spacing: first derivative lags by half a spacing -> small, bounded error
    assert worst < 3.0
    lin = TaylorForecaster(interval=4, max_order=1, first_enhance=2)
    for step in range(9):
        if lin.wants_model(step):
            lin.update(step, torch.tensor([3.0 * step]))
        else:
            assert abs(float(lin.forecast(step)) - 3.0 * step) < 1e-6  # a line is forecast exactly
    torch.manual_seed(2)
    model = create_model_from_config("bagel", dict(BASE, layer_module="Qwen2MoTDecoderLayer")).eval()
    with torch.no_grad():
        model.llm2vae.weight.normal_(0, 0.05)
    calls = []
    handle = model.llm2vae.register_forward_hook(lambda *a: calls.append(1))
    prompt = torch.randint(0, 100, (5,))
    kw = dict(boi_id=101, eoi_id=102, num_timesteps=16, noise_level=0.0)
    plain = model.generate_image(prompt, (2, 2), generator=torch.Generator().manual_seed(5), **kw)
    n_plain = len(calls)
    fast = model.generate_image(prompt, (2, 2), generator=torch.Generator().manual_seed(5), taylor={"interval": 3, "max_order": 2}, **kw)
    handle.remove()
    assert n_plain == 15 and len(calls) - n_plain == 8  # steps 0-4, 7, 10 and 13 of the 15
    scale = float(plain["image_latent"].abs().mean())
    assert float((fast["image_latent"] - plain["image_latent"]).abs().mean()) < 0.05 * scale
    every = model.generate_image(prompt, (2, 2), generator=torch.Generator().manual_seed(5), taylor={"interval": 1}, **kw)
    assert torch.equal(every["image_latent"], plain["image_latent"])


def test_conversation_kept_as_keys_and_values_matches_the_packed_stream():
    """Text, a clean condition image and more text appended turn by turn give the hidden states of one packed pass under
    the split rules; an image sampled after that conversation equals the one sampled from the same stream as a prompt."""
    from lmms_engine_b200.mapping_func import create_model_from_config
    from lmms_engine_b200.models.bagel import BagelContext

    torch.manual_seed(3)
    model = create_model_from_config("bagel", dict(BASE, layer_module="Qwen2MoTDecoderLayer")).eval()
    with torch.no_grad():
        model.llm2vae.weight.normal_(0, 0.05)
    t1, t2 = torch.randint(0, 100, (6,)), torch.randint(0, 100, (5,))
    lat = torch.randn(4, 16)
    side = model.config.max_latent_size
    lat_pos = (torch.arange(2)[:, None] * side + torch.arange(2)[None]).flatten()
    ctx = model.add_text(None, t1)
    ctx = model.add_image(ctx, 101, 102, latent_tokens=lat, latent_pos=lat_pos)
    ctx = model.add_text(ctx, t2)
    assert isinstance(ctx, BagelContext) and ctx.length == 6 + 6 + 5 and ctx.next_pos == 6 + 1 + 5
    ids = torch.cat([t1, torch.tensor([101, 0, 0, 0, 0, 102]), t2])
    pos = torch.cat([torch.arange(6), torch.full((6,), 6), torch.arange(7, 12)])
    with torch.no_grad():
        emb, _, _, _ = model.embed_stream(ids, lat, torch.arange(7, 11), lat_pos, torch.zeros(4), noise=torch.zeros(4, 16))
        cu = torch.tensor([0, 17], dtype=torch.int32)
        full = model.run_decoder(emb, pos, cu, torch.arange(7, 11), [6, 6, 5], ["causal", "full", "causal"])
    assert torch.allclose(ctx.last_hidden, full[12:], atol=2e-5), float((ctx.last_hidden - full[12:]).abs().max())
    after = model.generate_image(None, (2, 2), boi_id=101, eoi_id=102, num_timesteps=4, noise_level=0.0, context=ctx,
                                 generator=torch.Generator().manual_seed(9))
    # the same conversation as a plain text prompt (no image in between) must differ, the same text-only context must not
    text_ctx = model.add_text(None, torch.cat([t1, t2]))
    a = model.generate_image(None, (2, 2), boi_id=101, eoi_id=102, num_timesteps=4, noise_level=0.0, context=text_ctx,
                             generator=torch.Generator().manual_seed(9))
    b = model.generate_image(torch.cat([t1, t2]), (2, 2), boi_id=101, eoi_id=102, num_timesteps=4, noise_level=0.0,
                             generator=torch.Generator().manual_seed(9))
    assert torch.allclose(a["image_latent"], b["image_latent"], atol=2e-5)
    assert not torch.allclose(after["image_latent"], b["image_latent"], atol=1e-5)  # the condition image is seen
