"""Wan video family: text and image encoders against the transformers classes, the causal autoencoders' streaming
properties, the diffusion transformer against a plain restatement (complex rotary pairs), and the wrapper."""
import math
import os
import sys

import pytest
import torch
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def test_text_encoder_matches_umt5():
    from transformers import UMT5Config, UMT5EncoderModel

    from lmms_engine_b200.models.wan_encoders import WanTextEncoder

    torch.manual_seed(0)
    cfg = UMT5Config(vocab_size=100, d_model=32, d_kv=8, d_ff=64, num_layers=2, num_heads=4, relative_attention_num_buckets=32,
                     relative_attention_max_distance=128, feed_forward_proj="gated-gelu", dropout_rate=0.0)
    hf = UMT5EncoderModel(cfg).eval()
    with torch.no_grad():
        for p in hf.parameters():
            p.normal_(0, 0.3)
    enc = WanTextEncoder(vocab=100, dim=32, dim_attn=32, dim_ffn=64, num_heads=4, num_layers=2, num_buckets=32, shared_pos=False).eval()
    sd = {"token_embedding.weight": hf.state_dict()["shared.weight"], "norm.weight": hf.state_dict()["encoder.final_layer_norm.weight"]}
    for i in range(2):
        s, d = f"encoder.block.{i}.layer.", f"blocks.{i}."
        for a, b in (("0.SelfAttention.q", "attn.q"), ("0.SelfAttention.k", "attn.k"), ("0.SelfAttention.v", "attn.v"), ("0.SelfAttention.o", "attn.o"),
                     ("1.DenseReluDense.wi_0", "ffn.gate.0"), ("1.DenseReluDense.wi_1", "ffn.fc1"), ("1.DenseReluDense.wo", "ffn.fc2")):
            sd[d + b + ".weight"] = hf.state_dict()[s + a + ".weight"]
        sd[d + "norm1.weight"] = hf.state_dict()[s + "0.layer_norm.weight"]
        sd[d + "norm2.weight"] = hf.state_dict()[s + "1.layer_norm.weight"]
        sd[d + "pos_embedding.embedding.weight"] = hf.state_dict()[s + "0.SelfAttention.relative_attention_bias.weight"]
    missing, unexpected = enc.load_state_dict(sd, strict=True), None
    ids = torch.randint(0, 100, (2, 11))
    mask = torch.ones(2, 11, dtype=torch.long)
    mask[1, 7:] = 0
    with torch.no_grad():
        want = hf(input_ids=ids, attention_mask=mask).last_hidden_state
        got = enc(ids, mask)
        emb = enc.encode_prompt(ids, mask)
    assert (got[0] - want[0]).abs().max() < 1e-4 and (got[1, :7] - want[1, :7]).abs().max() < 1e-4
    assert float(emb[1, 7:].abs().sum()) == 0.0 and torch.equal(emb[0], got[0])


def test_image_encoder_matches_clip_vision():
    from transformers import CLIPVisionConfig, CLIPVisionModel

    from lmms_engine_b200.models.wan_encoders import CLIP_MEAN, CLIP_STD, WanImageEncoder

    torch.manual_seed(0)
    cfg = CLIPVisionConfig(hidden_size=32, intermediate_size=128, num_hidden_layers=3, num_attention_heads=4, image_size=28, patch_size=14,
                           hidden_act="gelu", layer_norm_eps=1e-5, attn_implementation="eager")
    hf = CLIPVisionModel(cfg).eval()
    with torch.no_grad():
        for p in hf.parameters():
            p.normal_(0, 0.2)
    enc = WanImageEncoder(image_size=28, patch_size=14, dim=32, mlp_ratio=4, out_dim=16, num_heads=4, num_layers=3).eval()
    h = {k[len("vision_model."):]: v for k, v in hf.state_dict().items()}
    sd = {"patch_embedding.weight": h["embeddings.patch_embedding.weight"], "cls_embedding": h["embeddings.class_embedding"].view(1, 1, -1),
          "pos_embedding": h["embeddings.position_embedding.weight"][None], "pre_norm.weight": h["pre_layrnorm.weight"],
          "pre_norm.bias": h["pre_layrnorm.bias"], "post_norm.weight": h["post_layernorm.weight"], "post_norm.bias": h["post_layernorm.bias"]}
    for i in range(3):
        s, d = f"encoder.layers.{i}.", f"transformer.{i}."
        sd[d + "attn.to_qkv.weight"] = torch.cat([h[s + f"self_attn.{n}_proj.weight"] for n in "qkv"], 0)
        sd[d + "attn.to_qkv.bias"] = torch.cat([h[s + f"self_attn.{n}_proj.bias"] for n in "qkv"], 0)
        for a, b in (("self_attn.out_proj", "attn.proj"), ("layer_norm1", "norm1"), ("layer_norm2", "norm2"), ("mlp.fc1", "mlp.0"), ("mlp.fc2", "mlp.2")):
            sd[d + b + ".weight"], sd[d + b + ".bias"] = h[s + a + ".weight"], h[s + a + ".bias"]
    missing, unexpected = enc.model.visual.load_state_dict(sd, strict=False)
    assert missing == ["head"] and not unexpected
    img = torch.rand(2, 3, 40, 40) * 2 - 1
    with torch.no_grad():
        got = enc.encode_image([img])
        x = F.interpolate(img, size=(28, 28), mode="bicubic", align_corners=False)
        x = ((x * 0.5 + 0.5) - torch.tensor(CLIP_MEAN).view(1, 3, 1, 1)) / torch.tensor(CLIP_STD).view(1, 3, 1, 1)
        want = hf(pixel_values=x, output_hidden_states=True).hidden_states[-2]  # all blocks but the last
    assert got.shape == (2, 5, 32) and (got - want).abs().max() < 1e-4


@pytest.mark.parametrize("variant", ["wan2.1", "wan2.2"])
def test_autoencoders_are_causal_and_follow_the_frame_rules(variant):
    from lmms_engine_b200.models.wan_vae import WanVAE

    torch.manual_seed(0)
    vae = WanVAE(variant, dim=8, z_dim=4, **({"dec_dim": 8} if variant == "wan2.2" else {}))
    with torch.no_grad():
        for p in vae.parameters():
            p.normal_(0, 0.3)
    assert not any(p.requires_grad for p in vae.parameters()) and not vae.model.training
    s = vae.upsampling_factor
    x = torch.rand(1, 3, 9, 32, 32) * 2 - 1
    z = vae.encode(x)
    assert z.shape == (1, 4, 3, 32 // s, 32 // s)  # T -> 1 + (T - 1) / 4
    # causal: the latents of the first 1 + 4j frames do not depend on later frames; a single frame is an image
    assert (vae.encode(x[:, :, :5]) - z[:, :, :2]).abs().max() < 1e-5
    assert (vae.encode(x[:, :, :1]) - z[:, :, :1]).abs().max() < 1e-5
    assert (vae.encode([x[0]]) - z).abs().max() < 1e-6
    lat = torch.randn(1, 4, 3, 32 // s, 32 // s)
    y = vae.model.decode(lat, vae.mean, vae.inv_std)
    assert y.shape == (1, 3, 9, 32, 32)  # T -> 1 + 4 (T - 1)
    y2 = vae.model.decode(lat[:, :, :2], vae.mean, vae.inv_std)
    assert (y2 - y[:, :, :5]).abs().max() < 1e-4
    assert (vae.model.decode(lat[:, :, :1], vae.mean, vae.inv_std) - y[:, :, :1]).abs().max() < 1e-4
    # checkpoint layout: the slots of the released implementation
    keys = set(vae.state_dict())
    if variant == "wan2.1":
        for k in ("model.encoder.conv1.weight", "model.encoder.downsamples.0.residual.2.weight", "model.encoder.downsamples.2.resample.1.weight",
                  "model.encoder.downsamples.5.time_conv.weight", "model.encoder.middle.1.to_qkv.weight", "model.encoder.head.0.gamma",
                  "model.decoder.upsamples.3.time_conv.weight", "model.decoder.upsamples.4.shortcut.weight", "model.conv1.weight", "model.conv2.bias"):
            assert k in keys, k
        assert len(vae.mean) == 4
    else:
        for k in ("model.encoder.downsamples.0.downsamples.0.residual.0.gamma", "model.encoder.downsamples.1.downsamples.2.time_conv.weight",
                  "model.decoder.upsamples.0.upsamples.3.resample.1.weight", "model.decoder.head.2.weight"):
            assert k in keys, k


def test_fold_and_shortcuts_of_the_48_channel_autoencoder():
    from lmms_engine_b200.models.wan_vae import AvgDown3D, DupUp3D, fold2x2, unfold2x2

    x = torch.arange(2 * 3 * 2 * 4 * 6, dtype=torch.float32).view(2, 3, 2, 4, 6)
    f = fold2x2(x)
    assert f.shape == (2, 12, 2, 2, 3) and torch.equal(unfold2x2(f), x)
    # channel order: (channel, column offset, row offset)
    assert float(f[0, 0, 0, 0, 0]) == float(x[0, 0, 0, 0, 0]) and float(f[0, 1, 0, 0, 0]) == float(x[0, 0, 0, 1, 0])
    assert float(f[0, 2, 0, 0, 0]) == float(x[0, 0, 0, 0, 1])
    down = AvgDown3D(4, 8, factor_t=2, factor_s=2)
    v = torch.rand(1, 4, 5, 4, 4)
    d = down(v)
    assert d.shape == (1, 8, 3, 2, 2)  # odd length: one zero frame is padded in FRONT
    up = DupUp3D(8, 4, factor_t=2, factor_s=2)
    u = up(d)
    assert u.shape == (1, 4, 5, 4, 4)  # the duplicate of the first frame is dropped


def _dit_reference(sd, cfg, x, t, ctx, heads):
    """One sample through the diffusion transformer with interleaved complex rotary pairs."""
    D, hd = cfg["dit_hidden_size"], cfg["dit_hidden_size"] // heads

    def lin(v, name):
        return v @ sd[name + ".weight"].T + sd[name + ".bias"]

    def rms(v, name):
        return v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + 1e-6) * sd[name + ".weight"]

    w = sd["patch_embedding.weight"]
    tok = F.conv3d(x[None], w, sd["patch_embedding.bias"], stride=w.shape[2:])
    f, h, wd = tok.shape[2:]
    tok = tok.flatten(2).transpose(1, 2)[0]
    pos = torch.cat([torch.cos(torch.outer(t.double(), torch.pow(10000, -torch.arange(128, dtype=torch.float64) / 128))),
                     torch.sin(torch.outer(t.double(), torch.pow(10000, -torch.arange(128, dtype=torch.float64) / 128)))], 1).float()
    te = lin(F.silu(lin(pos, "time_embedding.0")), "time_embedding.2")
    tm = lin(F.silu(te), "time_projection.1").view(1, 6, D)
    c = lin(F.gelu(lin(ctx, "text_embedding.0"), approximate="tanh"), "text_embedding.2")

    def freqs(n, d):
        fr = 1.0 / (10000 ** (torch.arange(0, d, 2)[: d // 2].double() / d))
        return torch.polar(torch.ones(n, d // 2, dtype=torch.float64), torch.outer(torch.arange(n).double(), fr))

    df = hd - 2 * (hd // 3)
    fc = torch.cat([freqs(f, df)[:, None, None].expand(f, h, wd, -1), freqs(h, hd // 3)[None, :, None].expand(f, h, wd, -1),
                    freqs(wd, hd // 3)[None, None].expand(f, h, wd, -1)], -1).reshape(f * h * wd, 1, -1)

    def rope(v):
        vc = torch.view_as_complex(v.double().view(v.shape[0], heads, hd // 2, 2))
        return torch.view_as_real(vc * fc).flatten(2).float()

    def attend(q, k, v):
        q, k, v = (u.view(u.shape[0], heads, hd).transpose(0, 1) for u in (q, k, v))
        return (torch.softmax(q @ k.transpose(1, 2) / math.sqrt(hd), -1) @ v).transpose(0, 1).reshape(-1, D)

    xs = tok
    for i in range(cfg["dit_num_layers"]):
        p = f"blocks.{i}."
        s1, c1, g1, s2, c2, g2 = (sd[p + "modulation"] + tm)[0]
        y = F.layer_norm(xs, (D,)) * (1 + c1) + s1
        q, k = rope(rms(lin(y, p + "self_attn.q"), p + "self_attn.norm_q").view(-1, heads, hd)), rope(rms(lin(y, p + "self_attn.k"), p + "self_attn.norm_k").view(-1, heads, hd))
        xs = xs + g1 * lin(attend(q.reshape(-1, D), k.reshape(-1, D), lin(y, p + "self_attn.v")), p + "self_attn.o")
        y = F.layer_norm(xs, (D,), sd[p + "norm3.weight"], sd[p + "norm3.bias"], 1e-6)
        a = attend(rms(lin(y, p + "cross_attn.q"), p + "cross_attn.norm_q"), rms(lin(c, p + "cross_attn.k"), p + "cross_attn.norm_k"), lin(c, p + "cross_attn.v"))
        xs = xs + lin(a, p + "cross_attn.o")
        y = F.layer_norm(xs, (D,)) * (1 + c2) + s2
        xs = xs + g2 * lin(F.gelu(lin(y, p + "ffn.0"), approximate="tanh"), p + "ffn.2")
    sh, sc = (sd["head.modulation"] + te[:, None])[0]
    out = lin(F.layer_norm(xs, (D,)) * (1 + sc) + sh, "head.head")
    pt, ph, pw = w.shape[2:]
    return out.view(f, h, wd, pt, ph, pw, -1).permute(6, 0, 3, 1, 4, 2, 5).reshape(-1, f * pt, h * ph, wd * pw)


DIT = dict(dit_hidden_size=48, dit_num_layers=2, dit_num_heads=2, dit_intermediate_size=96, dit_in_channels=4, dit_out_channels=4,
           dit_text_dim=32, dit_freq_dim=256)


def test_diffusion_transformer_matches_restatement_with_complex_rotary():
    from lmms_engine_b200.mapping_func import create_model_from_config

    torch.manual_seed(0)
    model = create_model_from_config("wanvideo", dict(DIT)).eval()
    with torch.no_grad():
        for p in model.dit.parameters():
            p.normal_(0, 0.2)
    sd = {k: v.detach() for k, v in model.dit.state_dict().items()}
    x, ctx, t = torch.randn(2, 4, 3, 4, 6), torch.randn(2, 5, 32), torch.tensor([300.0, 700.0])
    with torch.no_grad():
        got = model.denoise(x, t, ctx)
        want = torch.stack([_dit_reference(sd, DIT, x[i], t[i:i + 1], ctx[i], 2) for i in range(2)])
    assert got.shape == x.shape and (got - want).abs().max() < 2e-4 * max(1.0, float(want.abs().max()))
    # released transformer checkpoints carry no child prefix
    conv = model.convert_hf_state_dict({"blocks.0.modulation": sd["blocks.0.modulation"], "vae.model.conv1.weight": torch.zeros(1)})
    assert set(conv) == {"dit.blocks.0.modulation", "vae.model.conv1.weight"}


def test_wrapper_trains_from_pixels_and_prompts_with_frozen_towers():
    from lmms_engine_b200.mapping_func import create_model_from_config

    torch.manual_seed(0)
    cfg = dict(DIT, dit_has_image_input=True, dit_in_channels=4 + 4 + 4, require_clip_embedding=True, require_vae_embedding=True, clip_dim=32,
               clip_tokens=5, vae=dict(variant="wan2.1", dim=8, z_dim=4),
               text_encoder=dict(vocab=50, dim=32, dim_attn=32, dim_ffn=64, num_heads=4, num_layers=1),
               image_encoder=dict(image_size=28, patch_size=14, dim=32, num_heads=4, num_layers=2, out_dim=16),
               motion_controller=True, vace=dict(vace_layers=[0], vace_in_dim=6), trainable_modules="dit,vace,motion_controller")
    model = create_model_from_config("wanvideo", cfg)
    model.train()
    assert model.dit.training and not model.vae.training and not model.text_encoder.training
    trainable = {n.split(".")[0] for n, p in model.named_parameters() if p.requires_grad}
    assert trainable == {"dit", "vace", "motion_controller"}
    video = torch.rand(2, 3, 5, 32, 32) * 2 - 1
    ids = torch.randint(0, 50, (2, 6))
    mask = torch.ones_like(ids)
    out = model(video=video, input_ids=ids, attention_mask=mask, input_image=video[:, :, 0], vace_context=torch.randn(2, 6, 2, 4, 4),
                motion_bucket_id=torch.tensor([3.0, 7.0]))
    assert out["noise_pred"].shape == (2, 4, 2, 4, 4) and torch.isfinite(out["loss"])
    out["loss"].backward()
    assert model.dit.blocks[0].self_attn.q.weight.grad.abs().sum() > 0 and model.vace.vace_blocks[0].after_proj.weight.grad is not None
    assert model.dit.img_emb.proj[1].weight.grad.abs().sum() > 0  # the CLIP tokens reach the image cross-attention
    # the clean first frame is excluded from the loss: changing the target there changes nothing
    torch.manual_seed(1)
    idx, noise = torch.tensor([100, 900]), torch.randn(2, 4, 2, 4, 4)
    lat = model.encode_video(video).float()
    with torch.no_grad():
        model.eval()
        a = model(latents=lat, input_ids=ids, attention_mask=mask, input_image=video[:, :, 0], timestep_index=idx, noise=noise)["loss"]
        noise2 = noise.clone()
        noise2[:, :, :1] += 5.0
        b = model(latents=lat, input_ids=ids, attention_mask=mask, input_image=video[:, :, 0], timestep_index=idx, noise=noise2)["loss"]
    assert abs(float(a) - float(b)) < 1e-6
    # a zero-initialised motion controller leaves the prediction unchanged
    with torch.no_grad():
        y = model.first_frame_condition(video[:, :, 0], 5)
        assert y.shape == (2, 8, 2, 4, 4) and float(y[:, :4, 0].min()) == 1.0 and float(y[:, :4, 1].max()) == 0.0
        p0 = model.denoise(lat, torch.tensor([500.0, 500.0]), model.encode_prompt(ids, mask), y=y)
        p1 = model.denoise(lat, torch.tensor([500.0, 500.0]), model.encode_prompt(ids, mask), y=y, motion_bucket_id=torch.tensor([9.0]))
    assert torch.equal(p0, p1)
    with pytest.raises(ValueError, match="no vae"):
        create_model_from_config("wanvideo", dict(DIT))(video=video, context=torch.randn(2, 5, 32))


def test_wan_trainer_from_a_video_file_through_the_vision_dataset(tmp_path):
    """The reference's recipe: ``vision`` dataset + ``wanvideo`` processor + ``wan_trainer``, raw frames and a caption in,
    flow-matching loss out; only the diffusion transformer moves."""
    cv2 = pytest.importorskip("cv2")
    import json

    import numpy as np

    from tests.test_trainers_cpu import _run

    path = str(tmp_path / "clip.mp4")
    wr = cv2.VideoWriter(path, cv2.VideoWriter_fourcc(*"mp4v"), 8.0, (48, 40))
    rng = np.random.default_rng(0)
    for i in range(12):
        wr.write(rng.integers(0, 255, (40, 48, 3), dtype=np.uint8))
    wr.release()
    rec = {"messages": [{"role": "user", "content": [{"type": "video_url", "video_url": {"url": path}}, {"type": "text", "text": "noise on a screen"}]}]}
    data = tmp_path / "d.jsonl"
    data.write_text("\n".join(json.dumps(rec) for _ in range(4)) + "\n")
    dataset = {"dataset_type": "vision", "dataset_format": "jsonl", "dataset_path": str(data), "packing": False, "shuffle": False,
               "video_sampling_strategy": "frame_num", "frame_num": 5,
               "processor_config": {"processor_name": "byte", "processor_type": "wanvideo",
                                    "extra_kwargs": {"size": {"height": 32, "width": 32}}},
               "extra_kwargs": {"collator_type": "vision"}}
    cfg = dict(DIT, vae=dict(variant="wan2.1", dim=8, z_dim=4), text_encoder=dict(vocab=400, dim=32, dim_attn=32, dim_ffn=64, num_heads=4, num_layers=1),
               trainable_modules="dit")
    hist, runner = _run(tmp_path, "wan_trainer", "wanvideo", cfg, dataset, steps=2, per_device_train_batch_size=2)
    model = runner.trainer.model
    assert not any(p.requires_grad for p in model.vae.parameters()) and not model.text_encoder.training
    assert all(p.requires_grad for p in model.dit.parameters())
