"""The multimodal families on the GPU path (bf16, native kernels) against the same weights on CPU in fp32."""
import copy

import pytest
import torch

pytestmark = pytest.mark.gpu

TEXT = dict(vocab_size=256, hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=32)


def _compare(model_type, cfg, batch, tol=0.08):
    from lmms_engine_b200.mapping_func import create_model_from_config
    from lmms_engine_b200.ops import _cuda

    torch.manual_seed(0)
    ref = create_model_from_config(model_type, cfg).float()
    gpu = copy.deepcopy(ref).to("cuda", torch.bfloat16)
    loss_ref = ref(**batch)["loss"]
    loss_ref.backward()
    n0 = _cuda.launch_count
    moved = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in batch.items()}
    moved = {k: (v.to(torch.bfloat16) if torch.is_tensor(v) and v.is_floating_point() else v) for k, v in moved.items()}
    loss = gpu(**moved)["loss"]
    loss.backward()
    torch.cuda.synchronize()
    _cuda.check_status()
    assert _cuda.launch_count > n0, "the native kernels did not run"
    assert abs(float(loss) - float(loss_ref)) < tol, (float(loss), float(loss_ref))
    # a parameter deep inside the encoder received a finite gradient of the right scale
    for (n, p), (_, q) in zip(gpu.named_parameters(), ref.named_parameters()):
        if p.grad is None:
            continue
        assert torch.isfinite(p.grad).all(), n
    return gpu


def test_nanovlm_gpu():
    cfg = dict(text_config=TEXT, vision_config=dict(hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=2,
                                                    patch_size=8, num_patches=16), image_token_id=255)
    ids = torch.randint(0, 250, (96,))
    ids[5:21], ids[40:46] = 255, 255
    _compare("nanovlm", cfg, dict(input_ids=ids, labels=ids, cu_seqlens=torch.tensor([0, 30, 96], dtype=torch.int32),
                                  pixel_values=torch.randn(22, 3 * 64), spatial_shapes=torch.tensor([[4, 4], [2, 3]])))


def test_audio_families_gpu():
    enc = dict(num_mel_bins=32, d_model=128, encoder_layers=2, encoder_attention_heads=2, encoder_ffn_dim=256, max_source_positions=100)
    x = torch.randn(2, 32, 200)
    mask = (torch.arange(200)[None] < torch.tensor([200, 120])[:, None]).long()
    ids = torch.randint(0, 250, (120,))
    ids[3:53], ids[60:90] = 255, 255  # 50 + 30 pooled rows
    batch = dict(input_ids=ids, labels=ids, cu_seqlens=torch.tensor([0, 58, 120], dtype=torch.int32), input_features=x, feature_attention_mask=mask)
    _compare("qwen2_audio", dict(text_config=TEXT, audio_config=enc, audio_token_index=255), batch)
    omni = dict(model_type="qwen2_5_omni_audio_encoder", n_window=50, output_dim=64, **enc)
    _compare("aero", dict(text_config=TEXT, audio_config=omni, audio_token_index=255), batch)


def test_omni_thinkers_gpu():
    vis = dict(depth=2, hidden_size=128, intermediate_size=256, num_heads=2, patch_size=8, temporal_patch_size=2, spatial_merge_size=2,
               out_hidden_size=128, window_size=32, fullatt_block_indexes=[1])
    aud = dict(num_mel_bins=32, d_model=128, encoder_layers=1, encoder_attention_heads=2, encoder_ffn_dim=256, max_source_positions=100, n_window=50)
    text = dict(TEXT, mrope_section=[4, 6, 6])
    ids = torch.randint(0, 240, (100,))
    ids[3:7], ids[20:70] = 250, 252
    clips = torch.randn(1, 32, 200)
    batch = dict(input_ids=ids, labels=ids, cu_seqlens=torch.tensor([0, 100], dtype=torch.int32), pixel_values=torch.randn(16, 3 * 2 * 64),
                 image_grid_thw=torch.tensor([[1, 4, 4]]), audio_values=clips, audio_attention_mask=torch.ones(1, 200, dtype=torch.long))
    _compare("qwen2_5_omni_thinker", dict(text_config=text, vision_config=vis, audio_config=aud, image_token_index=250, video_token_index=251,
                                          audio_token_index=252), batch)


def test_llava_onevision_gpu():
    from lmms_engine_b200.models.llava_ov import anyres_grid, packed_image_tokens

    pins = [[32, 32], [32, 64], [64, 32], [64, 64]]
    cfg = dict(text_config=dict(TEXT, model_type="qwen2"), vision_config=dict(hidden_size=144, intermediate_size=256, num_hidden_layers=2,
                                                                           num_attention_heads=2, image_size=32, patch_size=8),
               image_token_index=250, video_token_index=251, image_grid_pinpoints=pins)
    size = (40, 60)
    n = packed_image_tokens(size, pins, 32, 4)
    tiles = 1 + anyres_grid(size, pins, 32)[0] * anyres_grid(size, pins, 32)[1]
    ids = torch.randint(0, 240, (20 + n,))
    ids[4:4 + n] = 250
    _compare("llava_onevision", cfg, dict(input_ids=ids, labels=ids, cu_seqlens=torch.tensor([0, 20 + n], dtype=torch.int32),
                                          pixel_values=torch.randn(tiles, 3, 32, 32), image_sizes=torch.tensor([list(size)])))


@pytest.mark.parametrize("linear_dim", [32, 128])  # 128: the state recurrence runs in its CUDA kernels
def test_qwen3_5_hybrid_gpu(linear_dim):
    cfg = dict(TEXT, num_hidden_layers=4, head_dim=64, linear_conv_kernel_dim=4, linear_key_head_dim=linear_dim,
               linear_value_head_dim=linear_dim, linear_num_key_heads=2, linear_num_value_heads=4, partial_rotary_factor=0.25)
    ids = torch.randint(0, 250, (200,))
    _compare("qwen3_5_text", cfg, dict(input_ids=ids, labels=ids, cu_seqlens=torch.tensor([0, 70, 200], dtype=torch.int32)))


def test_llava_onevision1_5_gpu():
    cfg = dict(model_type="llavaonevision1_5", text_config=dict(TEXT, rms_norm_eps=1e-6),
               vision_config=dict(depth=2, hidden_size=128, intermediate_size=256, num_heads=4, patch_size=8, text_hidden_size=128),
               image_token_id=250, video_token_id=251)
    ids = torch.randint(0, 240, (1, 64))
    ids[0, 4:10], ids[0, 30:34] = 250, 251
    grid_i, grid_v = torch.tensor([[1, 4, 6]]), torch.tensor([[2, 2, 4]])
    _compare("llavaonevision1_5", cfg, dict(input_ids=ids, attention_mask=torch.ones_like(ids), labels=ids,
                                            pixel_values=torch.randn(24, 3 * 8 * 8), image_grid_thw=grid_i,
                                            pixel_values_videos=torch.randn(16, 3 * 8 * 8), video_grid_thw=grid_v))


def test_gated_deltanet_matches_library_model_gpu():
    """Same weights in the FLA library's model (its Triton kernels) and in the native one: equal loss.  The
    comparison runs in a child process; if the library cannot be imported or its kernels fail there, the test
    skips with the child's message (the native model is covered by the CPU parity tests either way)."""
    import json
    import os
    import subprocess
    import sys

    helper = os.path.join(os.path.dirname(__file__), "helpers", "fla_parity_run.py")
    res = subprocess.run([sys.executable, helper], capture_output=True, text=True, timeout=900)
    if res.returncode != 0:
        tail = (res.stderr or res.stdout).strip().splitlines()[-1:] or ["no output"]
        if "lmms_engine_b200" in res.stderr and "fla" not in res.stderr.lower() and "triton" not in res.stderr.lower():
            raise AssertionError(res.stderr[-2000:])
        pytest.skip(f"library comparison did not run: {tail[0][:200]}")
    out = json.loads(res.stdout.strip().splitlines()[-1])
    assert out["native_launches"] > 0, "the native kernels did not run"
    assert abs(out["native"] - out["library"]) < 0.03, out


def test_qwen3_5_hybrid_step_time_report():
    """With ``QWEN35_TIME`` set: forward + backward of a four-layer hybrid stack at production head sizes
    (hidden 2048, 16 key / 32 value heads of 128, gated attention with 16 heads of 128) on 16 384 packed tokens."""
    import os

    if not os.environ.get("QWEN35_TIME"):
        pytest.skip("timing report only")
    from lmms_engine_b200.mapping_func import create_model_from_config

    torch.manual_seed(0)
    cfg = dict(vocab_size=32000, hidden_size=2048, intermediate_size=6144, num_hidden_layers=4, num_attention_heads=16,
               num_key_value_heads=4, head_dim=128, linear_conv_kernel_dim=4, linear_key_head_dim=128, linear_value_head_dim=128,
               linear_num_key_heads=16, linear_num_value_heads=32, partial_rotary_factor=0.25)
    model = create_model_from_config("qwen3_5_text", cfg).to("cuda", torch.bfloat16)
    lengths = [8192, 4096, 2048, 1024, 512, 256, 128, 128]
    ids = torch.randint(0, 32000, (sum(lengths),), device="cuda")
    cu = torch.tensor([0] + list(torch.tensor(lengths).cumsum(0).tolist()), dtype=torch.int32, device="cuda")
    for it in range(3):
        if it == 1:
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
        loss = model(input_ids=ids, labels=ids, cu_seqlens=cu)["loss"]
        loss.backward()
    b.record()
    torch.cuda.synchronize()
    assert torch.isfinite(loss)
    print(f"QWEN35_TIME 4 layers (3 linear-attention + 1 gated-attention), 16384 tokens: {a.elapsed_time(b) / 2:.1f} ms per forward+backward, "
          f"peak memory {torch.cuda.max_memory_allocated() / 2**30:.1f} GiB", flush=True)


def test_llava_onevision2_gpu():
    from lmms_engine_b200.models.llava_ov2 import build_patch_positions

    cfg = dict(model_type="llava_onevision2", text_config=dict(TEXT, rms_norm_eps=1e-6),
               vision_config=dict(depth=2, hidden_size=128, intermediate_size=256, num_heads=4, patch_size=8, spatial_merge_size=2,
                                  text_hidden_size=128, hidden_act="gelu"), image_token_id=250, video_token_id=251)
    ids = torch.randint(0, 240, (1, 64))
    ids[0, 4:10], ids[0, 30:33] = 250, 250
    grid = torch.tensor([[1, 4, 6], [3, 2, 2]])  # an image and three kept codec blocks
    import numpy as np

    pos = torch.from_numpy(np.concatenate([build_patch_positions([(1, 4, 6)], 2),
                                           np.array([[t, h, w] for t in (1, 4, 6) for h in (2, 3) for w in (0, 1)])]))
    _compare("llava_onevision2", cfg, dict(input_ids=ids, attention_mask=torch.ones_like(ids), labels=ids, pixel_values=torch.randn(36, 3 * 8 * 8),
                                           image_grid_thw=grid, patch_positions=pos))


def test_wanvideo_transformer_gpu():
    cfg = dict(dit_hidden_size=128, dit_num_layers=2, dit_num_heads=4, dit_intermediate_size=256, dit_in_channels=8, dit_out_channels=8,
               dit_text_dim=64, vace=dict(vace_layers=[0], vace_in_dim=6), motion_controller=True, trainable_modules="dit,vace,motion_controller")
    torch.manual_seed(1)
    lat = torch.randn(2, 8, 3, 8, 8)
    _compare("wanvideo", cfg, dict(latents=lat, context=torch.randn(2, 7, 64), timestep_index=torch.tensor([200, 800]),
                                   noise=torch.randn(2, 8, 3, 8, 8), vace_context=torch.randn(2, 6, 3, 8, 8),
                                   motion_bucket_id=torch.tensor([2.0, 5.0])), tol=0.2)


def test_rae_siglip_gpu():
    cfg = dict(noise_tau=0.0, encoder_config=dict(hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                                                  image_size=32, patch_size=8),
               decoder_config=dict(decoder_hidden_size=128, decoder_num_hidden_layers=2, decoder_num_attention_heads=4, decoder_intermediate_size=256))
    _compare("rae_siglip", cfg, dict(pixel_values=torch.rand(3, 3, 32, 32)))


def test_bagel_mixture_of_transformers_gpu():
    cfg = dict(TEXT, model_type="bagel", layer_module="Qwen2MoTDecoderLayer", qk_norm=True, attention_bias=True, latent_channels=4,
               latent_patch_size=2, max_latent_size=8, visual_und=True, vit_rope=False, vit_select_layer=-1, vit_max_num_patch_per_side=4,
               vit_config=dict(hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4, image_size=32, patch_size=8))
    from lmms_engine_b200.models.bagel_parts import flattened_position_ids

    ids = torch.randint(0, 250, (60,))
    batch = dict(input_ids=ids, labels=ids, cu_seqlens=torch.tensor([0, 36, 60], dtype=torch.int32), vit_tokens=torch.randn(8, 3 * 8 * 8),
                 vit_index=torch.arange(2, 10), vit_position_ids=flattened_position_ids(16, 32, 8, 4), vit_seqlens=torch.tensor([8]),
                 latent_tokens=torch.randn(6, 16), latent_index=torch.arange(20, 26), latent_pos=torch.tensor([0, 1, 2, 8, 9, 10]),
                 timesteps=torch.full((6,), 0.4), noise=torch.randn(6, 16),
                 split_lens=[2, 8, 10, 6, 10, 24], attn_modes=["causal", "full", "causal", "noise", "causal", "causal"])
    _compare("bagel", cfg, batch, tol=0.2)


def test_generation_on_cached_keys_gpu():
    """Prefill, then single-token steps against the key / value cache on the varlen kernel (one query row per sequence,
    keys of different lengths): hidden states of the full pass, within bf16 noise; the Bagel sampler on recorded prompt
    keys gives the image of the full-stream sampler."""
    from lmms_engine_b200.mapping_func import create_model_from_config
    from lmms_engine_b200.models.kv_cache import PackedKVCache
    from lmms_engine_b200.ops import _cuda

    torch.manual_seed(0)
    model = create_model_from_config("qwen3", dict(TEXT, model_type="qwen3", max_position_embeddings=512)).to("cuda", torch.bfloat16).eval()
    lens = [70, 33, 130]
    seqs = [torch.randint(0, 256, (n,), device="cuda") for n in lens]
    with torch.no_grad():
        cu = torch.tensor([0, 70, 103, 233], dtype=torch.int32, device="cuda")
        full = model(input_ids=torch.cat(seqs), cu_seqlens=cu)["hidden_states"].float()
        cache = PackedKVCache(2, [n + 4 for n in lens], device="cuda")
        heads = [n - 3 for n in lens]
        pos = cache.advance(heads)
        cu_h = torch.tensor([0, 67, 97, 224], dtype=torch.int32, device="cuda")
        out = [model(input_ids=torch.cat([s[:h] for s, h in zip(seqs, heads)]), cu_seqlens=cu_h, position_ids=pos, kv_cache=cache)["hidden_states"].float()]
        for step in range(3):
            pos = cache.advance([1, 1, 1])
            ids = torch.stack([s[h + step] for s, h in zip(seqs, heads)])
            out.append(model(input_ids=ids, cu_seqlens=torch.tensor([0, 1, 2, 3], dtype=torch.int32, device="cuda"), position_ids=pos,
                             kv_cache=cache)["hidden_states"].float())
    torch.cuda.synchronize()
    _cuda.check_status()
    at = 0
    for i, (n, h) in enumerate(zip(lens, heads)):
        start = [0, 67, 97][i]
        got = torch.cat([out[0][start:start + h]] + [out[1 + s][i:i + 1] for s in range(3)])
        ref = full[at:at + n]
        assert (got - ref).abs().max() < 0.06 * ref.abs().max(), (i, float((got - ref).abs().max()), float(ref.abs().max()))
        at += n
    bagel = create_model_from_config("bagel", dict(TEXT, model_type="bagel", latent_channels=4, latent_patch_size=2, max_latent_size=8,
                                                   attention_bias=True, layer_module="Qwen2MoTDecoderLayer")).to("cuda", torch.bfloat16).eval()
    prompt = torch.randint(0, 200, (40,), device="cuda")
    runs = [bagel.generate_image(prompt, (4, 4), boi_id=201, eoi_id=202, num_timesteps=4, noise_level=0.0, use_cache=flag,
                                 generator=torch.Generator("cuda").manual_seed(3)) for flag in (True, False)]
    torch.cuda.synchronize()
    _cuda.check_status()
    a, b = runs[0]["image_latent"].float(), runs[1]["image_latent"].float()
    assert torch.isfinite(a).all() and (a - b).abs().max() < 0.05 * b.abs().max() + 0.05


def test_audio_encoder_stream_gpu():
    """The streaming audio encoder on the varlen kernel: a few query frames against the cached keys of the left window
    (bottom-right aligned causal mask plus sliding window) gives the rows of the one-piece pass, within bf16 noise."""
    from lmms_engine_b200.models.audio import VoxtralRealtimeEncoder, VoxtralRealtimeEncoderConfig
    from lmms_engine_b200.ops import _cuda

    torch.manual_seed(0)
    cfg = VoxtralRealtimeEncoderConfig.from_dict(dict(hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=2,
                                                      head_dim=64, num_mel_bins=16, sliding_window=24))
    enc = VoxtralRealtimeEncoder(cfg).to("cuda", torch.bfloat16).eval()
    clip = torch.randn(1, 16, 400, device="cuda", dtype=torch.bfloat16)
    with torch.no_grad():
        whole = enc(clip)["last_hidden_state"].float()
        cache = enc.new_stream()
        cuts = [0, 8, 16, 64, 72, 200, 208, 400]
        rows = torch.cat([enc.stream(clip[0, :, a:b], cache) for a, b in zip(cuts[:-1], cuts[1:])]).float()
    torch.cuda.synchronize()
    _cuda.check_status()
    assert rows.shape == whole.shape == (200, 128)
    assert (rows - whole).abs().max() < 0.06 * whole.abs().max(), float((rows - whole).abs().max())
