"""LLaVA-OneVision-2: codec patch selection, the position-carrying tower, the processor and the streaming dataset."""
import json
import math

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from lmms_engine_b200.datasets.codec_video import positions_to_block_layout, select_codec_patches


def _video(n=6, H=32, W=48, seed=0):
    rng = np.random.default_rng(seed)
    base = rng.integers(0, 255, (H, W, 3), dtype=np.uint8)
    frames = np.stack([base.copy() for _ in range(n)])
    frames[2, 8:16, 16:24] = 255 - frames[2, 8:16, 16:24]  # one 8x8 block changes at t=2 and stays
    frames[3:, 8:16, 16:24] = frames[2, 8:16, 16:24]
    frames[5, 24:32, 0:8] = rng.integers(0, 255, (8, 8, 3), dtype=np.uint8)
    return frames


def test_codec_selection_keeps_key_frames_and_changed_blocks():
    frames = _video()
    out = select_codec_patches(frames, patch=4, merge=2, keyframe_interval=4, threshold=4.0, canvas_blocks=(4, 4), fps=2.0)
    gh, gw = 4, 6
    # frames 0 and 4 whole, one block at t=2, one at t=5
    assert out.kept_blocks == 2 * gh * gw + 2 and out.total_blocks == 6 * gh * gw
    pos = out.patch_positions
    used = pos[pos[:, 0] >= 0]
    assert used.shape[0] == out.kept_blocks * 4
    assert sorted(set(used[:, 0].tolist())) == [0, 2, 4, 5]
    at2 = used[used[:, 0] == 2]
    assert sorted(map(tuple, at2[:, 1:].tolist())) == [(2, 4), (2, 5), (3, 4), (3, 5)]
    # every kept patch on the canvases is the source patch at its position
    n_c, Hc, Wc, _ = out.canvases.shape
    grid = pos.reshape(n_c, Hc // 4, Wc // 4, 3)
    for c, i, j in [(0, 0, 0), (0, 3, 5), (n_c - 1, 0, 0)]:
        t, h, w = grid[c, i, j]
        if t < 0:
            continue
        assert (out.canvases[c, i * 4:(i + 1) * 4, j * 4:(j + 1) * 4] == frames[t, h * 4:(h + 1) * 4, w * 4:(w + 1) * 4]).all()
    assert np.allclose(out.source_pts, np.arange(6) / 2.0)
    # a block budget keeps the key frames and the largest residuals
    capped = select_codec_patches(frames, patch=4, merge=2, keyframe_interval=4, threshold=4.0, canvas_blocks=(4, 4), max_blocks=2 * gh * gw + 1)
    assert capped.kept_blocks == 2 * gh * gw + 1


def test_positions_to_block_layout_groups_merge_blocks():
    t, h, w = 1, 4, 4
    hh, ww = np.meshgrid(np.arange(h), np.arange(w), indexing="ij")
    pos = np.stack([np.zeros_like(hh), hh, ww], -1).reshape(-1, 3)
    out = positions_to_block_layout(pos, (t, h, w), 2)
    assert out[:4, 1:].tolist() == [[0, 0], [0, 1], [1, 0], [1, 1]]
    assert out[4:8, 1:].tolist() == [[0, 2], [0, 3], [1, 2], [1, 3]]


def _tower_reference(sd, patches, counts, pos, heads, merge, theta=10000.0):
    from lmms_engine_b200.models.llava_ov2 import rotary_sections

    def ln(x, p):
        return F.layer_norm(x, x.shape[-1:], sd[p + ".weight"], sd[p + ".bias"], 1e-5)

    x = patches @ sd["patch_embed.proj.weight"].reshape(sd["patch_embed.proj.weight"].shape[0], -1).T
    x = ln(x, "layernorm_pre")
    D = x.shape[1]
    hd = D // heads
    parts = []
    for axis, n in enumerate(rotary_sections(hd // 2)):
        invf = 1.0 / (theta ** (torch.arange(n, dtype=torch.float32) / max(n, 1)))
        parts.append(pos[:, axis:axis + 1].float() * invf[None])
    ang = torch.cat(parts, -1)
    cos, sin = torch.cat([ang, ang], -1).cos()[:, None], torch.cat([ang, ang], -1).sin()[:, None]

    def rot(v):
        a, b = v[..., : hd // 2], v[..., hd // 2:]
        return v * cos + torch.cat([-b, a], -1) * sin

    depth = len({k.split(".")[1] for k in sd if k.startswith("blocks.")})
    for i in range(depth):
        p = f"blocks.{i}."
        y = ln(x, p + "norm1")
        qkv = (y @ sd[p + "attn.qkv.weight"].T + sd[p + "attn.qkv.bias"]).view(-1, 3, heads, hd)
        q, k, v = rot(qkv[:, 0]), rot(qkv[:, 1]), qkv[:, 2]
        outs, s = [], 0
        for c in counts:
            a = torch.einsum("qhd,khd->hqk", q[s:s + c], k[s:s + c]) / math.sqrt(hd)
            outs.append(torch.einsum("hqk,khd->qhd", a.softmax(-1), v[s:s + c]).reshape(c, D))
            s += c
        x = x + torch.cat(outs) @ sd[p + "attn.proj.weight"].T + sd[p + "attn.proj.bias"]
        y = ln(x, p + "norm2")
        y = F.gelu(y @ sd[p + "mlp.fc1.weight"].T + sd[p + "mlp.fc1.bias"])
        x = x + y @ sd[p + "mlp.fc2.weight"].T + sd[p + "mlp.fc2.bias"]
    y = ln(x, "merger.ln_q").view(-1, D * merge * merge)
    y = F.gelu(y @ sd["merger.mlp.0.weight"].T + sd["merger.mlp.0.bias"])
    return y @ sd["merger.mlp.2.weight"].T + sd["merger.mlp.2.bias"]


TEXT = dict(vocab_size=300, hidden_size=48, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4,
            num_key_value_heads=2, head_dim=16, rms_norm_eps=1e-6, rope_theta=10000.0, max_position_embeddings=512,
            tie_word_embeddings=False)
VIS = dict(depth=2, hidden_size=64, intermediate_size=128, num_heads=4, patch_size=4, spatial_merge_size=2,
           text_hidden_size=48, hidden_act="gelu")


def _model():
    from lmms_engine_b200.mapping_func import create_model_from_config

    torch.manual_seed(0)
    model = create_model_from_config("llava_onevision2", dict(model_type="llava_onevision2", text_config=TEXT, vision_config=VIS,
                                                              image_token_id=290, video_token_id=291)).eval()
    with torch.no_grad():
        for p in model.visual.parameters():
            p.normal_(0, 0.1)
    return model


def test_tower_reads_rotary_angles_from_patch_positions():
    """The tower equals a plain restatement; an image given without positions gets the raster positions; a codec entry
    (a ragged set of blocks) is attended as one sequence with the source positions."""
    from lmms_engine_b200.models.llava_ov2 import build_patch_positions

    model = _model()
    assert type(model.visual).__name__ == "OneVisionTower"
    grid = torch.tensor([[1, 4, 6], [5, 2, 2]])  # an image and 5 kept codec blocks
    patches = torch.randn(24 + 20, 3 * 4 * 4)
    img_pos = build_patch_positions([(1, 4, 6)], 2)
    blocks = np.array([[0, 0, 0], [0, 2, 4], [3, 0, 2], [3, 2, 2], [7, 4, 0]])
    codec_pos = np.concatenate([[(t, h + di, w + dj) for di in range(2) for dj in range(2)] for t, h, w in blocks])
    pos = torch.from_numpy(np.concatenate([img_pos, codec_pos]))
    sd = {k: v.detach().float() for k, v in model.visual.state_dict().items()}
    with torch.no_grad():
        got = model.visual(patches, grid, pos)
        want = _tower_reference(sd, patches, [24, 20], pos, heads=4, merge=2)
        assert got.shape == (11, 48)
        assert (got - want).abs().max() < 3e-5
        only_image = model.visual(patches[:24], grid[:1])
        assert (only_image - got[:6]).abs().max() < 3e-5
        # positions matter (relatively, as rotary angles do): moving ONE codec block in time changes the codec entry only
        moved = pos.clone()
        moved[24:28, 0] += 3
        other = model.visual(patches, grid, moved)
        assert (other[:6] - got[:6]).abs().max() < 1e-6 and (other[6:] - got[6:]).abs().max() > 1e-4


def test_model_writes_features_over_placeholders_and_matches_hub_decoder():
    from transformers import Qwen3Config, Qwen3ForCausalLM

    model = _model()
    hf = Qwen3ForCausalLM(Qwen3Config(**TEXT, attn_implementation="eager")).eval().float()
    hub = {"model.language_model." + k[len("model."):] if k.startswith("model.") else k: v for k, v in hf.state_dict().items()}
    hub.update({"model.visual." + k: v for k, v in model.visual.state_dict().items()})
    missing, unexpected = model.load_state_dict(model.convert_hf_state_dict(hub), strict=False)
    assert not missing and not unexpected, (missing[:4], unexpected[:4])
    grid = torch.tensor([[1, 4, 6], [3, 2, 2]])
    patches = torch.randn(24 + 12, 3 * 4 * 4)
    from lmms_engine_b200.models.llava_ov2 import build_patch_positions

    pos = torch.from_numpy(np.concatenate([build_patch_positions([(1, 4, 6)], 2),
                                           np.array([[t, h, w] for t in (1, 4, 6) for h in (2, 3) for w in (0, 1)])]))
    ids = torch.randint(0, 280, (1, 40))
    ids[0, 3:9], ids[0, 20:23] = 290, 290
    with torch.no_grad():
        feats = model.visual(patches, grid, pos)
        emb = hf.model.embed_tokens(ids).clone()
        emb[0, 3:9], emb[0, 20:23] = feats[:6], feats[6:]
        ref = hf(inputs_embeds=emb, labels=ids).loss
        got = model(input_ids=ids, attention_mask=torch.ones_like(ids), labels=ids, pixel_values=patches,
                    image_grid_thw=grid, patch_positions=pos)["loss"]
    assert abs(float(ref) - float(got)) < 2e-5, (float(ref), float(got))
    # trains: gradients reach the tower through the placeholders
    model.train()
    out = model(input_ids=ids, attention_mask=torch.ones_like(ids), labels=ids, pixel_values=patches, image_grid_thw=grid, patch_positions=pos)
    out["loss"].backward()
    assert model.visual.blocks[0].attn.qkv.weight.grad.abs().sum() > 0


def _processor():
    from lmms_engine_b200.datasets.processor.llava_ov2_processor import LlavaOnevision2Processor
    from lmms_engine_b200.datasets.config import ProcessorConfig

    return LlavaOnevision2Processor(ProcessorConfig(processor_name="byte", processor_type="llava_onevision2",
                                                    extra_kwargs=dict(patch_size=4, merge_size=2, min_pixels=64, max_pixels=4096))).build()


def test_processor_aliases_codec_videos_into_the_image_path():
    from PIL import Image

    proc = _processor()
    frames = _video()
    codec = select_codec_patches(frames, patch=4, merge=2, keyframe_interval=4, threshold=4.0, canvas_blocks=(4, 4), fps=2.0)
    img = Image.fromarray(np.random.default_rng(1).integers(0, 255, (24, 40, 3), dtype=np.uint8))
    messages = [{"role": "user", "content": [{"type": "video"}, {"type": "text", "text": "what changes?"}, {"type": "image"}]},
                {"role": "assistant", "content": [{"type": "text", "text": "a block"}]}]
    out = proc.process(messages, images=[img], videos=[codec.canvases], video_metadata=[codec])
    grid = out["image_grid_thw"].tolist()
    # the video comes first in the text, so its entry comes first; it holds the kept blocks only
    assert grid[0] == [codec.kept_blocks, 2, 2]
    assert grid[1][0] == 1
    n_patches = sum(t * h * w for t, h, w in grid)
    assert out["pixel_values"].shape == (n_patches, 3 * 4 * 4) and out["patch_positions"].shape == (n_patches, 3)
    assert int((out["input_ids"] == proc.image_token_id).sum()) == n_patches // 4
    assert int((out["input_ids"] == proc.video_token_id).sum()) == 0
    assert (out["patch_positions"] >= 0).all()
    vid_pos = out["patch_positions"][: codec.kept_blocks * 4]
    assert sorted(set(vid_pos[:, 0].tolist())) == [0, 2, 4, 5]
    # the four patches of a merge block are adjacent
    blk = vid_pos.view(-1, 4, 3)
    assert (blk[:, :, 0] == blk[:, :1, 0]).all() and ((blk[:, 3, 1:] - blk[:, 0, 1:]) == 1).all()
    # the duration note precedes the placeholders, and only the answer is supervised
    text = bytes(t for t in out["input_ids"].tolist() if t < 256).decode(errors="ignore")
    assert "<2.5 seconds, 6 frames>" in text
    sup = out["labels"] != -100
    assert 0 < int(sup.sum()) < 20

    # a plainly sampled video (no codec metadata) keeps every patch of every frame
    plain = proc.process([{"role": "user", "content": [{"type": "video"}]}, {"role": "assistant", "content": "ok"}], videos=[frames])
    t, h, w = plain["image_grid_thw"][0].tolist()
    assert t == 6 and plain["patch_positions"][:, 0].max() == 5 and plain["pixel_values"].shape[0] == t * h * w


def test_streaming_dataset_feeds_codec_videos(tmp_path):
    cv2 = pytest.importorskip("cv2")
    import lmms_engine_b200.datasets.registry  # noqa: F401
    from lmms_engine_b200.mapping_func import DATASET_MAPPING
    from lmms_engine_b200.datasets.config import DatasetConfig

    frames = _video(n=8, H=32, W=48)
    path = str(tmp_path / "clip.mp4")
    wr = cv2.VideoWriter(path, cv2.VideoWriter_fourcc(*"mp4v"), 4.0, (48, 32))
    for f in frames:
        wr.write(cv2.cvtColor(f, cv2.COLOR_RGB2BGR))
    wr.release()
    rec = {"messages": [{"role": "user", "content": [{"type": "video_url", "video_url": {"url": path}}, {"type": "text", "text": "describe"}]},
                        {"role": "assistant", "content": [{"type": "text", "text": "noise"}]}]}
    data = tmp_path / "d.jsonl"
    data.write_text(json.dumps(rec) + "\n")
    cfg = DatasetConfig(dataset_type="llava_ov2_iterable", dataset_format="jsonl", dataset_path=str(data), packing=False, fps=4,
                        processor_config={"processor_name": "byte", "processor_type": "llava_onevision2",
                                          "extra_kwargs": dict(patch_size=4, merge_size=2)},
                        extra_kwargs={"codec": dict(patch_size=4, merge_size=2, keyframe_interval=4, threshold=12.0, canvas_blocks=(4, 4))})
    ds = DATASET_MAPPING["llava_ov2_iterable"](cfg)
    ds.build()
    sample = next(iter(ds))
    sample = sample[0] if isinstance(sample, (list, tuple)) else sample
    n = sample["pixel_values"].shape[0]
    assert sample["patch_positions"].shape == (n, 3) and n % 4 == 0
    assert int((sample["input_ids"] == ds.processor.image_token_id).sum()) == n // 4
    batch = ds.get_collator()([sample])
    assert "patch_positions" in batch and batch["patch_positions"].shape == (n, 3)
