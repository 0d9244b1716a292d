"""Parity of the native vision towers and the multimodal rotary index builder with the
upstream ``transformers`` implementations (fp32, CPU, random weights copied by name)."""
import os
import sys

import pytest
import torch
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
transformers = pytest.importorskip("transformers")


def _copy(src, dst):
    sd = {k: v for k, v in src.state_dict().items()}
    missing, unexpected = dst.load_state_dict(sd, strict=False)
    assert not missing and not unexpected, (missing[:5], unexpected[:5])


def test_qwen2_5_vl_tower_matches_hf():
    from transformers.models.qwen2_5_vl.configuration_qwen2_5_vl import Qwen2_5_VLVisionConfig
    from transformers.models.qwen2_5_vl.modeling_qwen2_5_vl import Qwen2_5_VisionTransformerPretrainedModel

    from lmms_engine_b200.models.vision import Qwen25VisionTower, VisionConfig

    kw = dict(depth=4, hidden_size=64, intermediate_size=96, num_heads=4, patch_size=14, out_hidden_size=48,
              window_size=56, fullatt_block_indexes=[1, 3], spatial_merge_size=2, temporal_patch_size=2, in_channels=3)
    torch.manual_seed(0)
    hf = Qwen2_5_VisionTransformerPretrainedModel._from_config(Qwen2_5_VLVisionConfig(**kw), attn_implementation="eager").float().eval()
    mine = Qwen25VisionTower(VisionConfig.from_dict(kw)).float().eval()
    _copy(hf, mine)
    grid = torch.tensor([[1, 6, 10], [2, 4, 4], [1, 8, 8]])
    P = int((grid[:, 0] * grid[:, 1] * grid[:, 2]).sum())
    pix = torch.randn(P, 3 * 2 * 14 * 14)
    with torch.no_grad():
        ref = hf(pix, grid_thw=grid)
        ref = ref.pooler_output if hasattr(ref, "pooler_output") else ref
        out = mine(pix, grid)
    assert out.shape == ref.shape
    assert torch.allclose(out, ref, atol=2e-4, rtol=1e-3), (out - ref).abs().max()


def test_qwen3_vl_tower_matches_hf():
    from transformers.models.qwen3_vl.configuration_qwen3_vl import Qwen3VLVisionConfig
    from transformers.models.qwen3_vl.modeling_qwen3_vl import Qwen3VLVisionModel

    from lmms_engine_b200.models.vision import Qwen3VisionTower, VisionConfig

    kw = dict(depth=4, hidden_size=64, intermediate_size=96, num_heads=4, patch_size=16, out_hidden_size=48,
              spatial_merge_size=2, temporal_patch_size=2, in_channels=3, num_position_embeddings=64,
              deepstack_visual_indexes=[0, 2], hidden_act="gelu_pytorch_tanh")
    torch.manual_seed(0)
    hf = Qwen3VLVisionModel._from_config(Qwen3VLVisionConfig(**kw), attn_implementation="eager").float().eval()
    mine = Qwen3VisionTower(VisionConfig.from_dict(kw)).float().eval()
    _copy(hf, mine)
    grid = torch.tensor([[1, 6, 10], [2, 4, 4]])
    P = int((grid[:, 0] * grid[:, 1] * grid[:, 2]).sum())
    pix = torch.randn(P, 3 * 2 * 16 * 16)
    with torch.no_grad():
        ref = hf(pix, grid_thw=grid)
        if isinstance(ref, tuple):
            ref_main, ref_deep = ref[0], ref[1]
        else:
            ref_main, ref_deep = ref.pooler_output, ref.deepstack_features
        out, deep = mine(pix, grid)
    assert torch.allclose(out, ref_main, atol=2e-4, rtol=1e-3), (out - ref_main).abs().max()
    for a, b in zip(deep, ref_deep):
        assert torch.allclose(a, b, atol=2e-4, rtol=1e-3)


def _slow_mrope(ids, vision_ids, grids, seconds, merge, tps):
    """Token-by-token oracle of the documented rule (text advances all streams; a vision run
    takes temporal / row / column indices offset by the running position; text resumes at max+1)."""
    pos, cur, g, i = [], 0, 0, 0
    ids = list(ids)
    while i < len(ids):
        if ids[i] not in vision_ids:
            pos.append((cur, cur, cur))
            cur += 1
            i += 1
            continue
        t, h, w = grids[g]
        gh, gw = h // merge, w // merge
        block = []
        for f in range(t):
            for r in range(gh):
                for c in range(gw):
                    block.append((int(f * seconds[g] * tps) + cur, r + cur, c + cur))
        pos += block
        cur = max(max(p) for p in block) + 1
        i += len(block)
        g += 1
    return torch.tensor(pos).t()


def test_mrope_positions_match_slow_oracle():
    from lmms_engine_b200.models import mrope

    img, vid = [1, 4, 6], [3, 4, 4]
    doc1 = [1, 2, 252] + [250] * 6 + [5, 6, 252] + [251] * 12 + [7, 8, 9]
    doc2 = [3, 252] + [250] * 4 + [4]
    ids = torch.tensor(doc1 + doc2)
    cu = torch.tensor([0, len(doc1), len(doc1) + len(doc2)], dtype=torch.int32)
    grids, secs = [img, vid, [1, 4, 4]], [0.0, 1.5, 0.0]
    mine = mrope.build_mrope_positions(ids, cu, (250, 251), grids, secs, 2, 2.0)
    ref = torch.cat([_slow_mrope(doc1, (250, 251), grids[:2], secs[:2], 2, 2.0),
                     _slow_mrope(doc2, (250, 251), grids[2:], secs[2:], 2, 2.0)], 1)
    assert torch.equal(mine, ref)
    # temporal index of the third video frame: floor(2 * 1.5 s * 2 tokens/s) = 6 past the run start
    start = 3 + 6 + 3  # tokens before the video run in doc1
    assert mine[0, start + 2 * 4] - mine[0, start] == 6


def test_nanovlm_encodes_images_independently_and_trains():
    """Patches of different images never attend to each other; image features land on the placeholders;
    padded and packed inputs give the same loss."""
    from lmms_engine_b200.mapping_func import create_model_from_config

    cfg = dict(text_config=dict(vocab_size=128, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                                num_key_value_heads=2, head_dim=16),
               vision_config=dict(hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=2, patch_size=4,
                                  num_patches=16),
               image_token_id=127, projector_num_layers=2)
    torch.manual_seed(0)
    m = create_model_from_config("nanovlm", cfg)
    shapes = torch.tensor([[4, 4], [2, 3]])
    pix = torch.randn(22, 48)
    enc = m.vision_model
    with torch.no_grad():
        both, a, b = enc(pix, shapes), enc(pix[:16], shapes[:1]), enc(pix[16:], shapes[1:])
    assert torch.allclose(both, torch.cat([a, b]), atol=1e-5)
    ids = torch.randint(0, 120, (60,))
    ids[5:21] = 127
    ids[30:36] = 127
    cu = torch.tensor([0, 25, 60], dtype=torch.int32)
    out = m(input_ids=ids, labels=ids, cu_seqlens=cu, pixel_values=pix, spatial_shapes=shapes)
    out["loss"].backward()
    assert m.vision_model.patch_embedding.weight.grad.abs().sum() > 0
    # the same two documents as a padded batch
    padded = torch.zeros(2, 35, dtype=torch.long)
    mask = torch.zeros(2, 35, dtype=torch.long)
    padded[0, :25], mask[0, :25] = ids[:25], 1
    padded[1, :35], mask[1, :35] = ids[25:], 1
    out2 = m(input_ids=padded, labels=padded, attention_mask=mask, pixel_values=pix, spatial_shapes=shapes)
    assert abs(float(out["loss"]) - float(out2["loss"])) < 1e-5


def test_audio_encoder_matches_upstream_and_feeds_the_decoder():
    """Native Whisper-style encoder on valid frames only == upstream Qwen2AudioEncoder with its key mask;
    pooled features land on the audio placeholders of the packed stream."""
    pytest.importorskip("transformers")
    from transformers.models.qwen2_audio.configuration_qwen2_audio import Qwen2AudioEncoderConfig
    from transformers.models.qwen2_audio.modeling_qwen2_audio import Qwen2AudioEncoder

    from lmms_engine_b200.mapping_func import create_model_from_config
    from lmms_engine_b200.models.audio import AudioEncoder

    enc = dict(num_mel_bins=16, d_model=32, encoder_layers=2, encoder_attention_heads=4, encoder_ffn_dim=64, max_source_positions=20)
    torch.manual_seed(0)
    hf = Qwen2AudioEncoder(Qwen2AudioEncoderConfig(**enc)).eval()
    cfg = dict(text_config=dict(vocab_size=128, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                                num_key_value_heads=2, head_dim=16), audio_config=enc, audio_token_index=127)
    model = create_model_from_config("qwen2_audio", cfg)
    model.audio_tower.load_state_dict(hf.state_dict(), strict=True)
    x = torch.randn(2, 16, 40)
    lens = torch.tensor([40, 27])
    mask = (torch.arange(40)[None] < lens[:, None]).long()
    frames, out_len = AudioEncoder.output_lengths(lens)
    key_ok = torch.arange(20)[None] < frames[:, None]
    am = torch.zeros(2, 1, 20, 20).masked_fill(~key_ok[:, None, None, :], float("-inf"))
    with torch.no_grad():
        ref = hf(x, attention_mask=am).last_hidden_state
        got, ol = model.audio_tower(x, mask)
    assert ol.tolist() == out_len.tolist() == [10, 7]
    off = 0
    for i, m in enumerate(ol.tolist()):
        assert torch.allclose(got[off:off + m], ref[i, :m], atol=1e-5)
        off += m
    ids = torch.randint(0, 120, (50,))
    ids[3:13] = 127
    ids[30:37] = 127
    cu = torch.tensor([0, 20, 50], dtype=torch.int32)
    out = model(input_ids=ids, labels=ids, cu_seqlens=cu, input_features=x, feature_attention_mask=mask)
    out["loss"].backward()
    assert model.audio_tower.conv1.weight.grad.abs().sum() > 0 and model.multi_modal_projector.linear.weight.grad.abs().sum() > 0
    # the collator's names for the same tensors are accepted as well
    out2 = model(input_ids=ids, labels=ids, cu_seqlens=cu, audio_values=x, audio_attention_mask=mask)
    assert abs(float(out["loss"]) - float(out2["loss"])) < 1e-6


def test_omni_audio_encoder_matches_upstream():
    """Chunked audio encoder (attention inside 2*n_window-frame chunks) == upstream Qwen2_5OmniAudioEncoder."""
    pytest.importorskip("transformers")
    from transformers.models.qwen2_5_omni.configuration_qwen2_5_omni import Qwen2_5OmniAudioEncoderConfig
    from transformers.models.qwen2_5_omni.modeling_qwen2_5_omni import Qwen2_5OmniAudioEncoder

    from lmms_engine_b200.mapping_func import create_model_from_config
    from lmms_engine_b200.models.audio import OmniAudioEncoder, OmniAudioEncoderConfig

    kw = dict(num_mel_bins=16, d_model=32, encoder_layers=2, encoder_attention_heads=4, encoder_ffn_dim=64, max_source_positions=60,
              n_window=10, output_dim=24)
    torch.manual_seed(0)
    hc = Qwen2_5OmniAudioEncoderConfig(**kw)
    hc._attn_implementation = "eager"
    hf = Qwen2_5OmniAudioEncoder(hc).eval()
    mine = OmniAudioEncoder(OmniAudioEncoderConfig(**kw)).eval()
    mine.load_state_dict(hf.state_dict(), strict=True)
    lens = torch.tensor([47, 20, 33])
    x = torch.randn(16, int(lens.sum()))
    after, out_len = OmniAudioEncoder.output_lengths(lens)
    with torch.no_grad():
        ref = hf(x, feature_lens=lens, aftercnn_lens=after).last_hidden_state
        got, ol = mine(x, lens)
    assert ol.tolist() == out_len.tolist() and torch.allclose(got, ref, atol=1e-5)
    # aero with this encoder: padded clips in, features on the placeholders
    model = create_model_from_config("aero", dict(
        text_config=dict(vocab_size=128, hidden_size=64, intermediate_size=128, num_hidden_layers=1, num_attention_heads=4,
                         num_key_value_heads=2, head_dim=16),
        audio_config=dict(model_type="qwen2_5_omni_audio_encoder", **kw), audio_token_index=127))
    clips = torch.randn(2, 16, 50)
    mask = torch.zeros(2, 50, dtype=torch.long)
    mask[0, :47], mask[1, :20] = 1, 1
    ids = torch.randint(0, 120, (40,))
    ids[2:14], ids[20:25] = 127, 127  # 12 + 5 pooled rows
    out = model(input_ids=ids, labels=ids, cu_seqlens=torch.tensor([0, 40], dtype=torch.int32), audio_values=clips, audio_attention_mask=mask)
    out["loss"].backward()
    assert model.audio_tower.proj.weight.grad.abs().sum() > 0


def test_omni_thinker_matches_upstream_with_text_image_and_audio():
    """Hub-format weights load (separate q/k/v of the vision blocks are fused) and the loss equals the
    upstream Qwen2.5-Omni thinker on a sequence with an image and an audio clip."""
    pytest.importorskip("transformers")
    from transformers.models.qwen2_5_omni.configuration_qwen2_5_omni import Qwen2_5OmniThinkerConfig
    from transformers.models.qwen2_5_omni.modeling_qwen2_5_omni import Qwen2_5OmniThinkerForConditionalGeneration

    from lmms_engine_b200.mapping_func import create_model_from_config

    torch.manual_seed(0)
    text = dict(vocab_size=160, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                rope_scaling={"mrope_section": [2, 3, 3], "rope_type": "default", "type": "default"}, max_position_embeddings=512,
                rope_theta=10000.0)
    vis = dict(depth=2, hidden_size=32, intermediate_size=64, num_heads=2, patch_size=4, temporal_patch_size=2, spatial_merge_size=2,
               out_hidden_size=64, window_size=16, fullatt_block_indexes=[1], in_channels=3)
    aud = dict(num_mel_bins=16, d_model=32, encoder_layers=1, encoder_attention_heads=4, encoder_ffn_dim=64, max_source_positions=60,
               n_window=10, output_dim=64)
    hc = Qwen2_5OmniThinkerConfig(text_config=text, vision_config=vis, audio_config=aud, image_token_index=150, video_token_index=151,
                                  audio_token_index=152, position_id_per_seconds=25, audio_start_token_id=153, audio_end_token_id=154,
                                  vision_start_token_id=155, vision_end_token_id=156)
    for c in (hc, hc.text_config, hc.vision_config, hc.audio_config):
        c._attn_implementation = "eager"
    hf = Qwen2_5OmniThinkerForConditionalGeneration(hc).eval().float()
    mine = create_model_from_config("qwen2_5_omni_thinker", hc.to_dict()).eval()
    missing, unexpected = mine.load_state_dict(mine.convert_hf_state_dict(hf.state_dict()), strict=False)
    assert not missing and not unexpected
    ids = torch.randint(0, 140, (1, 50))
    ids[0, 2], ids[0, 3:7], ids[0, 7] = 155, 150, 156
    ids[0, 19], ids[0, 20:32], ids[0, 32] = 153, 152, 154
    pix, grid = torch.randn(16, 3 * 2 * 4 * 4), torch.tensor([[1, 4, 4]])
    clips = torch.randn(1, 16, 50)
    mask = torch.zeros(1, 50, dtype=torch.long)
    mask[0, :47] = 1
    kw = dict(input_ids=ids, attention_mask=torch.ones_like(ids), labels=ids, pixel_values=pix, image_grid_thw=grid,
              input_features=clips, feature_attention_mask=mask)
    with torch.no_grad():
        ref, got = hf(**kw).loss, mine(**kw)["loss"]
    assert abs(float(ref) - float(got)) < 1e-4, (float(ref), float(got))


def test_llava_onevision_matches_upstream_and_processor_counts():
    """Any-resolution packing (grid layout, un-padding, newline per row, base view first) and video pooling
    give the upstream loss on hub-format weights; the processor reserves exactly the rows the model produces."""
    pytest.importorskip("transformers")
    import numpy as np
    from PIL import Image
    from transformers.models.llava_onevision.configuration_llava_onevision import LlavaOnevisionConfig as HC
    from transformers.models.llava_onevision.modeling_llava_onevision import LlavaOnevisionForConditionalGeneration

    from lmms_engine_b200.datasets import registry  # noqa: F401
    from lmms_engine_b200.datasets.config import ProcessorConfig
    from lmms_engine_b200.mapping_func import DATAPROCESSOR_MAPPING, create_model_from_config
    from lmms_engine_b200.models.llava_ov import anyres_grid, packed_image_tokens

    torch.manual_seed(0)
    text = dict(model_type="qwen2", vocab_size=200, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                num_key_value_heads=2, max_position_embeddings=4096, rope_theta=10000.0)
    vis = dict(model_type="siglip_vision_model", hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=2,
               image_size=16, patch_size=4, vision_use_head=False)
    pins = [[16, 16], [16, 32], [32, 16], [32, 32], [16, 48], [48, 16]]
    hc = HC(text_config=text, vision_config=vis, image_token_index=190, video_token_index=191, image_grid_pinpoints=pins,
            vision_aspect_ratio="anyres_max_9", tie_word_embeddings=False)
    for c in (hc, hc.text_config, hc.vision_config):
        c._attn_implementation = "eager"
    hf = LlavaOnevisionForConditionalGeneration(hc).eval().float()
    mine = create_model_from_config("llava_onevision", hc.to_dict()).eval()
    missing, unexpected = mine.load_state_dict(mine.convert_hf_state_dict(hf.state_dict()), strict=False)
    assert not missing and not unexpected
    sizes = [(30, 50), (40, 20)]
    ntoks = [packed_image_tokens(s, pins, 16, 4) for s in sizes]
    counts = [1 + anyres_grid(s, pins, 16)[0] * anyres_grid(s, pins, 16)[1] for s in sizes]
    pix = torch.randn(2, max(counts), 3, 16, 16)
    ids = torch.randint(0, 180, (1, 20 + sum(ntoks)))
    ids[0, 3:3 + ntoks[0]] = 190
    ids[0, 10 + ntoks[0]:10 + ntoks[0] + ntoks[1]] = 190
    kw = dict(input_ids=ids, attention_mask=torch.ones_like(ids), labels=ids, pixel_values=pix, image_sizes=torch.tensor(sizes))
    with torch.no_grad():
        assert abs(float(hf(**kw).loss) - float(mine(**kw)["loss"])) < 1e-4
    nv = 3 * 4 + 1
    idv = torch.randint(0, 180, (1, 10 + nv))
    idv[0, 2:2 + nv] = 191
    kv = dict(input_ids=idv, attention_mask=torch.ones_like(idv), labels=idv, pixel_values_videos=torch.randn(1, 3, 3, 16, 16))
    with torch.no_grad():
        assert abs(float(hf(**kv).loss) - float(mine(**kv)["loss"])) < 1e-4
    # processor: tiles in order, flattened over images; placeholder count == rows of the packed features
    proc = DATAPROCESSOR_MAPPING["llava_onevision"](ProcessorConfig(processor_name="none", processor_type="llava_onevision", extra_kwargs={
        "image_size": 16, "patch_size": 4, "image_grid_pinpoints": pins})).build()
    img = Image.fromarray((np.random.rand(30, 50, 3) * 255).astype("uint8"))
    out = proc.process([{"role": "user", "content": [{"type": "image"}, {"type": "text", "text": "what"}]},
                        {"role": "assistant", "content": [{"type": "text", "text": "a"}]}], images=[img])
    assert out["pixel_values"].shape == (counts[0], 3, 16, 16) and out["image_sizes"].tolist() == [[30, 50]]
    assert int((out["input_ids"] == proc.image_token_id).sum()) == ntoks[0]
    feats = mine.image_features(out["pixel_values"], out["image_sizes"])
    assert feats.shape[0] == ntoks[0]


def test_qwen3_omni_thinker_matches_upstream():
    """Mixture-of-experts decoder + deepstack vision tower + Qwen3-Omni audio encoder: hub-format weights load
    (patch-merger names are mapped) and text / image / audio losses equal the upstream thinker."""
    pytest.importorskip("transformers")
    from transformers.models.qwen3_omni_moe.configuration_qwen3_omni_moe import Qwen3OmniMoeThinkerConfig
    from transformers.models.qwen3_omni_moe.modeling_qwen3_omni_moe import Qwen3OmniMoeThinkerForConditionalGeneration

    from lmms_engine_b200.mapping_func import create_model_from_config
    from lmms_engine_b200.models.audio import omni3_output_lengths

    torch.manual_seed(0)
    text = dict(vocab_size=160, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                head_dim=16, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32, decoder_sparse_step=1, norm_topk_prob=True,
                mlp_only_layers=[], rope_scaling={"mrope_section": [2, 3, 3], "rope_type": "default", "mrope_interleaved": True},
                max_position_embeddings=512, rope_theta=10000.0, router_aux_loss_coef=0.0)
    vis = dict(depth=2, hidden_size=32, intermediate_size=64, num_heads=2, patch_size=4, temporal_patch_size=2, spatial_merge_size=2,
               out_hidden_size=64, num_position_embeddings=16, deepstack_visual_indexes=[0], in_channels=3)
    aud = dict(num_mel_bins=16, d_model=32, encoder_layers=1, encoder_attention_heads=4, encoder_ffn_dim=64, max_source_positions=100,
               n_window=50, n_window_infer=200, output_dim=64, downsample_hidden_size=8, conv_chunksize=3)
    hc = Qwen3OmniMoeThinkerConfig(text_config=text, vision_config=vis, audio_config=aud, image_token_id=150, video_token_id=151,
                                   audio_token_id=152, position_id_per_seconds=13, audio_start_token_id=153, vision_start_token_id=155)
    for c in (hc, hc.text_config, hc.vision_config, hc.audio_config):
        c._attn_implementation = "eager"
    hf = Qwen3OmniMoeThinkerForConditionalGeneration(hc).eval().float()
    mine = create_model_from_config("qwen3_omni_moe_thinker", hc.to_dict()).eval()
    missing, unexpected = mine.load_state_dict(mine.convert_hf_state_dict(hf.state_dict()), strict=False)
    assert not missing and not unexpected

    def same(**kw):
        kw.update(attention_mask=torch.ones_like(kw["input_ids"]), labels=kw["input_ids"])
        with torch.no_grad():
            a, b = float(hf(**kw).loss), float(mine(**kw)["loss"])
        assert abs(a - b) < 1e-4, (a, b)

    t = torch.randint(0, 140, (1, 50))
    same(input_ids=t)
    ti = t.clone()
    ti[0, 2], ti[0, 3:7] = 155, 150
    same(input_ids=ti, pixel_values=torch.randn(16, 3 * 2 * 4 * 4), image_grid_thw=torch.tensor([[1, 4, 4]]))
    clips = torch.randn(1, 16, 100)
    mask = torch.zeros(1, 100, dtype=torch.long)
    mask[0, :90] = 1  # one attention window: the upstream eager path ignores window boundaries, the flash path and this one do not
    n = int(omni3_output_lengths(torch.tensor([90]))[0])
    ta = t.clone()
    ta[0, 19], ta[0, 20:20 + n] = 153, 152
    same(input_ids=ta, input_features=clips, feature_attention_mask=mask)


def test_voxtral_realtime_encoder_matches_upstream():
    """Causal convolutions + rotary sliding-window attention == upstream VoxtralRealtimeEncoder; a right-padded clip
    gives the same frames as the clip alone."""
    pytest.importorskip("transformers")
    from transformers.models.voxtral_realtime.configuration_voxtral_realtime import VoxtralRealtimeEncoderConfig as HC
    from transformers.models.voxtral_realtime.modeling_voxtral_realtime import VoxtralRealtimeEncoder as HF

    from lmms_engine_b200.mapping_func import create_model_from_config

    torch.manual_seed(0)
    hc = HC(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, head_dim=16, num_mel_bins=16, sliding_window=12)
    hc._attn_implementation = "eager"
    hf = HF(hc).eval()
    mine = create_model_from_config("voxtral_realtime_encoder", hc.to_dict()).eval()
    mine.load_state_dict(hf.state_dict(), strict=True)
    x = torch.randn(2, 16, 60)
    with torch.no_grad():
        ref = hf(input_features=x).last_hidden_state
        got = mine(x)["last_hidden_state"].view(2, 30, 64)
    assert torch.allclose(got, ref, atol=1e-4)
    mask = torch.ones(2, 60, dtype=torch.long)
    mask[1, 41:] = 0
    with torch.no_grad():
        out = mine(x, mask)
    assert out["frame_lengths"].tolist() == [30, 20]  # frame 20 would also cover mel frame 41, outside the clip
    assert torch.allclose(out["last_hidden_state"][30:], ref[1, :20], atol=1e-4)


def test_gated_delta_rule_chunked_equals_recurrent():
    from lmms_engine_b200.models.qwen3_5 import chunk_gated_delta_rule, recurrent_gated_delta_rule

    torch.manual_seed(0)
    for T in (1, 63, 64, 150):
        q, k, v = torch.randn(T, 3, 16), torch.randn(T, 3, 16), torch.randn(T, 3, 24)
        g, beta = -torch.rand(T, 3) * 0.5, torch.rand(T, 3)
        assert torch.allclose(chunk_gated_delta_rule(q, k, v, g, beta), recurrent_gated_delta_rule(q, k, v, g, beta), atol=1e-5)


@pytest.mark.parametrize("moe", [False, True])
def test_qwen3_5_hybrid_decoder_matches_upstream(moe):
    """Gated-DeltaNet + gated-attention hybrid (dense and mixture-of-experts) == upstream on hub-format weights;
    two packed documents == the two documents alone (state and convolution never cross the boundary)."""
    pytest.importorskip("transformers")
    from lmms_engine_b200.mapping_func import create_model_from_config

    torch.manual_seed(0)
    kw = dict(vocab_size=200, hidden_size=64, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2, head_dim=32,
              linear_conv_kernel_dim=4, linear_key_head_dim=16, linear_value_head_dim=16, linear_num_key_heads=2, linear_num_value_heads=4,
              max_position_embeddings=512, rope_parameters={"rope_theta": 10000.0, "partial_rotary_factor": 0.25, "rope_type": "default"},
              tie_word_embeddings=False)
    if moe:
        from transformers.models.qwen3_5_moe.configuration_qwen3_5_moe import Qwen3_5MoeTextConfig as HC
        from transformers.models.qwen3_5_moe.modeling_qwen3_5_moe import Qwen3_5MoeForCausalLM as HF

        kw.update(moe_intermediate_size=32, shared_expert_intermediate_size=48, num_experts=4, num_experts_per_tok=2, router_aux_loss_coef=0.0)
        name = "qwen3_5_moe_text"
    else:
        from transformers.models.qwen3_5.configuration_qwen3_5 import Qwen3_5TextConfig as HC
        from transformers.models.qwen3_5.modeling_qwen3_5 import Qwen3_5ForCausalLM as HF

        kw.update(intermediate_size=128)
        name = "qwen3_5_text"
    hc = HC(**kw)
    hc._attn_implementation = "eager"
    hf = HF(hc).eval().float()
    for n, p in hf.named_parameters():
        if "norm" in n and "linear_attn" not in n:
            torch.nn.init.normal_(p, std=0.1)  # zero-centred scales: make them matter
    mine = create_model_from_config(name, hc.to_dict()).eval()
    missing, unexpected = mine.load_state_dict(mine.convert_hf_state_dict(hf.state_dict()), strict=False)
    assert not missing and not unexpected
    ids = torch.randint(0, 200, (1, 90))
    with torch.no_grad():
        ref = float(hf(input_ids=ids, labels=ids).loss)
        got = float(mine(input_ids=ids, attention_mask=torch.ones_like(ids), labels=ids)["loss"])
        a, b = ids[0, :50], ids[0, 50:]
        la, lb = float(hf(input_ids=a[None], labels=a[None]).loss), float(hf(input_ids=b[None], labels=b[None]).loss)
        packed = float(mine(input_ids=ids[0], labels=ids[0], cu_seqlens=torch.tensor([0, 50, 90], dtype=torch.int32))["loss"])
    assert abs(ref - got) < 1e-4, (ref, got)
    assert abs((la * 49 + lb * 39) / 88 - packed) < 1e-4


def test_qwen3_5_vision_language_wrapper_matches_upstream():
    """``qwen3_5`` as an image-text model: Qwen3-VL style tower without deepstack, interleaved M-RoPE on the
    rotary half of the gated-attention layers, hybrid decoder; loss equal to the hub model's."""
    from transformers.models.qwen3_5 import modeling_qwen3_5 as m
    from transformers.models.qwen3_5.configuration_qwen3_5 import Qwen3_5Config

    from lmms_engine_b200.mapping_func import create_model_from_config

    torch.manual_seed(0)
    text = dict(vocab_size=200, hidden_size=64, intermediate_size=128, num_hidden_layers=4, num_attention_heads=4,
                num_key_value_heads=2, head_dim=32, linear_conv_kernel_dim=4, linear_key_head_dim=16,
                linear_value_head_dim=16, linear_num_key_heads=2, linear_num_value_heads=4, max_position_embeddings=512,
                rope_parameters={"rope_theta": 10000.0, "partial_rotary_factor": 0.5, "rope_type": "default",
                                 "mrope_section": [2, 3, 3], "mrope_interleaved": True})
    vis = dict(depth=2, hidden_size=32, intermediate_size=64, num_heads=2, patch_size=4, temporal_patch_size=2,
               spatial_merge_size=2, out_hidden_size=64, num_position_embeddings=16, in_channels=3)
    hc = Qwen3_5Config(text_config=text, vision_config=vis, image_token_id=190, video_token_id=191,
                       vision_start_token_id=192, vision_end_token_id=193, tie_word_embeddings=False)
    for c in (hc, hc.text_config, hc.vision_config):
        c._attn_implementation = "eager"
    hf = m.Qwen3_5ForConditionalGeneration(hc).eval().float()
    mine = create_model_from_config("qwen3_5", hc.to_dict()).eval()
    assert type(mine).__name__ == "VLModel" and type(mine.language_model).__name__ == "Qwen35LM"
    missing, unexpected = mine.load_state_dict(mine.convert_hf_state_dict(hf.state_dict()), strict=False)
    assert not missing and not unexpected, (missing[:4], unexpected[:4])
    ids = torch.randint(0, 180, (1, 60))
    ids[0, 2], ids[0, 3:7], ids[0, 7] = 192, 190, 193
    pix, grid = torch.randn(16, 3 * 2 * 4 * 4), torch.tensor([[1, 4, 4]])
    mm = (ids == 190).long()
    ones = torch.ones_like(ids)
    with torch.no_grad():
        ref = hf(input_ids=ids, attention_mask=ones, labels=ids, pixel_values=pix, image_grid_thw=grid,
                 mm_token_type_ids=mm).loss
        got = mine(input_ids=ids, attention_mask=ones, labels=ids, pixel_values=pix, image_grid_thw=grid)["loss"]
        t = torch.randint(0, 180, (1, 60))
        ref_t = hf(input_ids=t, labels=t).loss
        got_t = mine(input_ids=t, attention_mask=torch.ones_like(t), labels=t)["loss"]
    assert abs(float(ref) - float(got)) < 2e-5, (float(ref), float(got))
    assert abs(float(ref_t) - float(got_t)) < 2e-5, (float(ref_t), float(got_t))


def _rice_reference(sd, patches, grid, heads, merge):
    """Plain fp32 restatement of the Rice tower for one packed batch: every frame is
    [class token, patches], attends within itself with 2-D rotary angles (learned for the class token)."""
    D = sd["pre_layernorm.weight"].numel()
    hd = D // heads
    x = patches @ sd["patch_embed.proj.weight"].reshape(D, -1).T
    invf = 1.0 / (10000.0 ** (torch.arange(0, hd // 2, 2, dtype=torch.float32) / (hd // 2)))
    outs, at = [], 0
    for t, h, w in grid:
        for _ in range(t):
            n = h * w
            rows = torch.arange(h).view(h // merge, merge, 1, 1).expand(h // merge, merge, w // merge, merge)
            cols = torch.arange(w).view(1, 1, w // merge, merge).expand(h // merge, merge, w // merge, merge)
            rows, cols = rows.permute(0, 2, 1, 3).reshape(-1), cols.permute(0, 2, 1, 3).reshape(-1)
            ang = torch.cat([rows[:, None] * invf, cols[:, None] * invf], -1)
            ang = torch.cat([sd["class_pos_emb"], ang], 0)
            ang = torch.cat([ang, ang], -1)
            cos, sin = ang.cos()[:, None], ang.sin()[:, None]
            y = torch.cat([sd["class_embedding"][None], x[at:at + n]], 0)
            at += n
            y = F.layer_norm(y, (D,), sd["pre_layernorm.weight"], sd["pre_layernorm.bias"], 1e-5)
            i = 0
            while f"blocks.{i}.norm1.weight" in sd:
                b = f"blocks.{i}."
                z = F.layer_norm(y, (D,), sd[b + "norm1.weight"], sd[b + "norm1.bias"], 1e-5)
                q, k, v = (z @ sd[b + "attn.qkv.weight"].T + sd[b + "attn.qkv.bias"]).view(-1, 3, heads, hd).unbind(1)
                rot = lambda u: u * cos + torch.cat([-u[..., hd // 2:], u[..., :hd // 2]], -1) * sin
                q, k = rot(q), rot(k)
                a = torch.softmax(torch.einsum("qhd,khd->hqk", q, k) / hd ** 0.5, -1)
                o = torch.einsum("hqk,khd->qhd", a, v).reshape(-1, D)
                y = y + o @ sd[b + "attn.proj.weight"].T + sd[b + "attn.proj.bias"]
                z = F.layer_norm(y, (D,), sd[b + "norm2.weight"], sd[b + "norm2.bias"], 1e-5)
                z = F.gelu(z @ sd[b + "mlp.fc1.weight"].T + sd[b + "mlp.fc1.bias"])
                y = y + z @ sd[b + "mlp.fc2.weight"].T + sd[b + "mlp.fc2.bias"]
                i += 1
            outs.append(y[1:])
    y = torch.cat(outs)
    y = F.layer_norm(y, (D,), sd["merger.ln_q.weight"], sd["merger.ln_q.bias"], 1e-5).view(-1, D * merge * merge)
    y = F.gelu(y @ sd["merger.mlp.0.weight"].T + sd["merger.mlp.0.bias"])
    return y @ sd["merger.mlp.2.weight"].T + sd["merger.mlp.2.bias"]


def test_llava_onevision1_5_rice_tower_and_decoder_wiring():
    """``llavaonevision1_5``: the Rice tower equals a plain restatement (several frames, a video), and the whole
    model's loss equals the hub Qwen3 decoder fed the same embeddings with plain 1-D positions."""
    from transformers import Qwen3Config, Qwen3ForCausalLM

    from lmms_engine_b200.mapping_func import create_model_from_config

    torch.manual_seed(0)
    text = dict(vocab_size=300, hidden_size=48, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4,
                num_key_value_heads=2, head_dim=16, rms_norm_eps=1e-6, rope_theta=10000.0, max_position_embeddings=256,
                tie_word_embeddings=False)
    vis = dict(depth=2, hidden_size=64, intermediate_size=128, num_heads=4, patch_size=4, spatial_merge_size=2,
               text_hidden_size=48, hidden_act="gelu", layer_norm_eps=1e-5)
    model = create_model_from_config("llavaonevision1_5", dict(model_type="llavaonevision1_5", text_config=text,
                                                               vision_config=vis, image_token_id=290, video_token_id=291)).eval()
    assert type(model.visual).__name__ == "RiceVisionTower"
    with torch.no_grad():
        for p in model.visual.parameters():
            p.normal_(0, 0.1)
    grid = torch.tensor([[1, 4, 6], [2, 2, 4]])
    patches = torch.randn(24 + 16, 3 * 4 * 4)
    sd = {k: v.detach().float() for k, v in model.visual.state_dict().items()}
    with torch.no_grad():
        feats = model.visual(patches, grid)
    want = _rice_reference(sd, patches, grid.tolist(), heads=4, merge=2)
    assert feats.shape == (10, 48)
    assert (feats - want).abs().max() < 2e-5
    # gradients reach the class token and its learned rotary angle
    model.visual(patches, grid).square().sum().backward()
    assert model.visual.class_pos_emb.grad.abs().sum() > 0 and model.visual.class_embedding.grad.abs().sum() > 0

    hf = Qwen3ForCausalLM(Qwen3Config(**text, attn_implementation="eager")).eval().float()
    hub = {"model.language_model." + k[len("model."):] if k.startswith("model.") else k: v for k, v in hf.state_dict().items()}
    hub.update({"model.visual." + k: v for k, v in model.visual.state_dict().items()})
    missing, unexpected = model.load_state_dict(model.convert_hf_state_dict(hub), strict=False)
    assert not missing and not unexpected, (missing[:4], unexpected[:4])
    ids = torch.randint(0, 280, (1, 40))
    ids[0, 3:9], ids[0, 20:24] = 290, 291
    with torch.no_grad():
        emb = hf.model.embed_tokens(ids).clone()
        emb[0, 3:9], emb[0, 20:24] = feats[:6], feats[6:]
        ref = hf(inputs_embeds=emb, labels=ids).loss
        got = model(input_ids=ids, attention_mask=torch.ones_like(ids), labels=ids, pixel_values=patches[:24],
                    image_grid_thw=grid[:1], pixel_values_videos=patches[24:], video_grid_thw=grid[1:])["loss"]
    assert abs(float(ref) - float(got)) < 2e-5, (float(ref), float(got))


def test_packed_gated_delta_rule_equals_per_document_rule_and_convolution():
    """All documents at once (padded to whole chunks, state reset per document) == one document at a time;
    the packed causal convolution == ``conv1d`` per document; gradients agree as well."""
    from lmms_engine_b200.models.qwen3_5 import chunk_gated_delta_rule
    from lmms_engine_b200.ops import gdn

    torch.manual_seed(0)
    lengths = [70, 5, 64, 130]
    T, H, dk, dv = sum(lengths), 3, 16, 8
    q, k, v = (torch.randn(T, H, d, requires_grad=True) for d in (dk, dk, dv))
    g = (-torch.rand(T, H)).requires_grad_()
    beta = torch.rand(T, H).requires_grad_()
    got = gdn.chunk_gated_delta_rule_packed(q, k, v, g, beta, lengths)
    want, at = [], 0
    for L in lengths:
        want.append(chunk_gated_delta_rule(q[at:at + L], k[at:at + L], v[at:at + L], g[at:at + L], beta[at:at + L]))
        at += L
    want = torch.cat(want)
    assert (got - want).abs().max() < 1e-5
    probe = torch.randn_like(got)
    ga = torch.autograd.grad((got * probe).sum(), (q, k, v, g, beta))
    gb = torch.autograd.grad((want * probe).sum(), (q, k, v, g, beta))
    for a, b in zip(ga, gb):
        assert (a - b).abs().max() < 1e-4 * max(1.0, float(b.abs().max()))
    x = torch.randn(T, 6)
    conv = torch.nn.Conv1d(6, 6, 4, groups=6, padding=3, bias=False)
    pos = torch.cat([torch.arange(L) for L in lengths])
    out = gdn.causal_conv_silu_packed(x, conv.weight[:, 0], pos)
    ref, at = [], 0
    for L in lengths:
        ref.append(F.silu(conv(x[at:at + L].t()[None])[0, :, :L]).t())
        at += L
    assert (out - torch.cat(ref)).abs().max() < 1e-6


@pytest.mark.parametrize("family", ["qwen3_vl", "qwen3_5"])
def test_aero_realtime_adds_audio_rows_to_the_text_stream(family):
    """Without audio and text stream the model IS its backbone; with them, the decoder sees the text-stream
    embeddings plus the projected audio rows at the audio positions (checked against a hand-built embedding)."""
    from lmms_engine_b200.mapping_func import create_model_from_config

    torch.manual_seed(0)
    text = dict(vocab_size=300, hidden_size=64, intermediate_size=128, num_hidden_layers=2 if family == "qwen3_vl" else 4,
                num_attention_heads=4, num_key_value_heads=2, head_dim=16, tie_word_embeddings=False)
    if family == "qwen3_5":
        text.update(linear_conv_kernel_dim=4, linear_key_head_dim=16, linear_value_head_dim=16, linear_num_key_heads=2,
                    linear_num_value_heads=4, rope_parameters={"rope_theta": 10000.0, "partial_rotary_factor": 0.5,
                                                               "mrope_section": [2, 1, 1], "mrope_interleaved": True})
    else:
        text.update(rope_scaling={"mrope_section": [4, 2, 2], "mrope_interleaved": True})
    vis = dict(depth=2, hidden_size=32, intermediate_size=64, num_heads=2, patch_size=4, temporal_patch_size=2, spatial_merge_size=2,
               out_hidden_size=64, num_position_embeddings=16, in_channels=3, deepstack_visual_indexes=[0] if family == "qwen3_vl" else [])
    audio = dict(hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=2, head_dim=16, num_mel_bins=8,
                 sliding_window=6)
    cfg = dict(model_type="aero_realtime", backbone_family=family, text_config=text, vision_config=vis, audio_config=audio,
               downsample_factor=2, image_token_index=290, video_token_index=291, audio_token_index=292,
               vision_start_token_index=293)
    model = create_model_from_config("aero_realtime", cfg).eval()
    assert type(model).__name__ == "AeroRealtimeModel" and model.config.to_dict()["backbone_family"] == family
    backbone = create_model_from_config(family, dict(model_type=family, text_config=text, vision_config=vis, image_token_id=290,
                                                     video_token_id=291, vision_start_token_id=293)).eval()
    missing, unexpected = backbone.load_state_dict(model.state_dict(), strict=False)
    assert not missing and all(k.startswith(("audio_tower.", "multi_modal_projector.")) for k in unexpected)
    ids = torch.randint(0, 280, (1, 48))
    ids[0, 2], ids[0, 3:7] = 293, 290
    ids[0, 20:25] = 292
    pix, grid = torch.randn(16, 3 * 2 * 4 * 4), torch.tensor([[1, 4, 4]])
    ones = torch.ones_like(ids)
    common = dict(input_ids=ids, attention_mask=ones, labels=ids, pixel_values=pix, image_grid_thw=grid)
    with torch.no_grad():
        plain = model(**common)["loss"]
        assert abs(float(plain) - float(backbone(**common)["loss"])) < 1e-6
        # two clips: 13 and 8 mel frames -> 6 and 4 encoder frames -> 3 + 2 rows of two frames each
        feats = torch.randn(2, 8, 13)
        mel_mask = torch.zeros(2, 13, dtype=torch.long)
        mel_mask[0, :13], mel_mask[1, :8] = 1, 1
        stream = ids.clone()
        stream[0, 20:25] = torch.tensor([281, 282, 283, 281, 281])
        got = model(**common, text_stream_ids=stream, input_features=feats, feature_attention_mask=mel_mask)["loss"]
        frame_mask = torch.zeros(2, 6, dtype=torch.long)
        frame_mask[0, :6], frame_mask[1, :4] = 1, 1
        again = model(**common, text_stream_ids=stream, input_features=feats, audio_attention_mask=frame_mask)["loss"]
        enc = model.audio_tower(feats, mel_mask)
        hidden = enc["last_hidden_state"]
        assert enc["frame_lengths"].tolist() == [6, 4]
        rows = torch.cat([hidden[0:6].reshape(3, -1), hidden[6:10].reshape(2, -1)])
        rows = model.multi_modal_projector(rows)
        emb, deep, deep_idx = VLModel_embed(model, ids[0], pix, grid, stream[0])
        emb[20:25] += rows
        lm = model.language_model
        _, labels, pos, cu, _ = lm.prepare_packed(ids, ones, ids, None, None)
        from lmms_engine_b200.models import mrope

        pos = mrope.build_mrope_positions(ids[0], cu, (290, 291), grid.tolist(), [0.0], 2, 0.0)
        want = lm(inputs_embeds=emb, labels=labels, position_ids=pos, cu_seqlens=cu, deepstack=deep, deepstack_index=deep_idx)["loss"]
    assert abs(float(got) - float(want)) < 1e-5 and abs(float(got) - float(plain)) > 1e-4
    assert abs(float(again) - float(got)) < 1e-6  # the same clips described by a frame-level mask


def VLModel_embed(model, ids, pix, grid, stream):
    from lmms_engine_b200.models.vl import VLModel

    return VLModel.embed_multimodal(model, ids, pix, grid, None, None, embed_ids=stream)


def test_gated_deltanet_lm_loads_library_checkpoints_and_matches_token_recurrence():
    """``gated_deltanet``: parameter names / shapes of the FLA library's model load strictly; one linear-attention
    layer equals a token-by-token restatement built from its weights (two documents, value heads = 2 x key heads)."""
    from lmms_engine_b200.mapping_func import create_model_from_config
    from lmms_engine_b200.models.decoder_lm import PackedContext
    from lmms_engine_b200.models.qwen3_5 import recurrent_gated_delta_rule

    torch.manual_seed(0)
    cfg = dict(vocab_size=200, hidden_size=64, num_hidden_layers=2, num_heads=2, num_v_heads=4, head_dim=16, expand_v=2.0, hidden_ratio=4)
    model = create_model_from_config("gated_deltanet", cfg).eval()
    assert model.config.intermediate_size == 256
    try:
        import warnings

        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            from fla.models import GatedDeltaNetConfig as FC, GatedDeltaNetForCausalLM as FM
        lib = FM(FC(**cfg, fuse_norm=False, fuse_swiglu=False))
        model.load_state_dict(model.convert_hf_state_dict(lib.state_dict()), strict=True)
    except ImportError:
        pass
    layer = model.model.layers[0].attn
    lens = [37, 70]
    x = torch.randn(sum(lens), 64)
    cu = torch.tensor([0, 37, 107], dtype=torch.int32)
    ctx = PackedContext(cu, 70, None, None, True)
    with torch.no_grad():
        got = layer(x, ctx)
        outs, at = [], 0
        for L in lens:
            seg = x[at:at + L]
            at += L

            def conv(t, w):  # causal depthwise convolution, last tap on the current token, then SiLU
                pad = F.pad(t, (0, 0, w.shape[-1] - 1, 0))
                return F.silu(sum(pad[j:j + L] * w[:, 0, j] for j in range(w.shape[-1])))

            q = conv(seg @ layer.q_proj.weight.T, layer.q_conv1d.weight).view(L, 2, 16).repeat_interleave(2, 1)
            k = conv(seg @ layer.k_proj.weight.T, layer.k_conv1d.weight).view(L, 2, 16).repeat_interleave(2, 1)
            v = conv(seg @ layer.v_proj.weight.T, layer.v_conv1d.weight).view(L, 4, 32)
            g = -layer.A_log.exp() * F.softplus(seg @ layer.a_proj.weight.T + layer.dt_bias)
            beta = (seg @ layer.b_proj.weight.T).sigmoid()
            o = recurrent_gated_delta_rule(q, k, v, g, beta)
            o = o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + 1e-6) * layer.o_norm.weight
            gate = (seg @ layer.g_proj.weight.T).view(L, 4, 32)
            outs.append((o * F.silu(gate)).reshape(L, -1) @ layer.o_proj.weight.T)
        want = torch.cat(outs)
    assert (got - want).abs().max() < 2e-5 * max(1.0, float(want.abs().max()))
    ids = torch.randint(0, 200, (107,))
    out = model(input_ids=ids, labels=ids, cu_seqlens=cu)
    out["loss"].backward()
    assert torch.isfinite(out["loss"]) and model.model.layers[1].attn.A_log.grad is not None


def test_omni_audio_in_video_positions_match_upstream():
    """Interleaved audio-visual blocks (``use_audio_in_video``): token order and ``(t, h, w)`` positions equal the
    upstream index of Qwen2.5-Omni, including stand-alone clips and images in the same stream."""
    pytest.importorskip("transformers")
    import numpy as np
    from transformers.models.qwen2_5_omni.configuration_qwen2_5_omni import Qwen2_5OmniThinkerConfig
    from transformers.models.qwen2_5_omni.modeling_qwen2_5_omni import Qwen2_5OmniThinkerForConditionalGeneration

    from lmms_engine_b200.models.mrope import interleave_av, omni_positions_one

    text = dict(vocab_size=200, hidden_size=32, intermediate_size=64, num_hidden_layers=1, num_attention_heads=2, num_key_value_heads=1,
                rope_scaling={"mrope_section": [2, 3, 3], "rope_type": "default", "type": "default"})
    vis = dict(depth=1, hidden_size=16, intermediate_size=32, num_heads=2, patch_size=4, temporal_patch_size=2, spatial_merge_size=2,
               out_hidden_size=32, window_size=16, fullatt_block_indexes=[0])
    aud = dict(num_mel_bins=8, d_model=16, encoder_layers=1, encoder_attention_heads=2, encoder_ffn_dim=32, max_source_positions=100,
               n_window=10, output_dim=32)
    IMG, VID, AUD, VS, VE, AS, AE = 150, 151, 152, 153, 154, 155, 156
    hc = Qwen2_5OmniThinkerConfig(text_config=text, vision_config=vis, audio_config=aud, image_token_index=IMG, video_token_index=VID,
                                  audio_token_index=AUD, vision_start_token_id=VS, vision_end_token_id=VE, audio_start_token_id=AS,
                                  audio_end_token_id=AE, position_id_per_seconds=25, seconds_per_chunk=2)
    upstream = Qwen2_5OmniThinkerForConditionalGeneration(hc)
    rng = np.random.default_rng(0)
    for trial in range(8):
        grid_v = [(int(rng.integers(2, 6)), 4, int(rng.choice([4, 8])))]
        spg = [float(rng.choice([1.0, 2.0, 0.5]))]
        mel = int(rng.integers(100, 900))
        n_a = ((mel - 1) // 2 + 1 - 2) // 2 + 1
        t, h, w = grid_v[0]
        vt = np.floor(np.repeat(np.arange(t), (h // 2) * (w // 2)) * spg[0] * 25).astype(np.int64)
        block = []
        for kind, lo, hi in interleave_av(vt, n_a, 50):
            block += [VID if kind == "video" else AUD] * (hi - lo)
        ids = [1, 2, 3, VS] + [IMG] * 4 + [VE, 5, 6, VS, AS] + block + [AE, VE, 7, 8, 9]
        mels = [mel]
        if trial % 2:
            ids += [AS] + [AUD] * 37 + [AE, 10, 11]
            mels.append(37 * 4)
        ids_t = torch.tensor([ids])
        ref, _ = upstream.get_rope_index(ids_t, torch.tensor([(1, 4, 4)]), torch.tensor(grid_v), torch.ones_like(ids_t), True,
                                         torch.tensor(mels), torch.tensor(spg))
        mine = omni_positions_one(np.array(ids), IMG, VID, AUD, [(1, 4, 4)], grid_v, spg, 2, 25.0, 2.0)
        assert np.array_equal(ref[:, 0].numpy(), mine), trial


def _tiny_realtime(family="qwen3_vl"):
    from lmms_engine_b200.mapping_func import create_model_from_config

    text = dict(vocab_size=300, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                head_dim=16, tie_word_embeddings=False, rope_scaling={"mrope_section": [4, 2, 2], "mrope_interleaved": True})
    vis = dict(depth=2, hidden_size=32, intermediate_size=64, num_heads=2, patch_size=4, temporal_patch_size=2, spatial_merge_size=2,
               out_hidden_size=64, num_position_embeddings=16, in_channels=3, deepstack_visual_indexes=[0])
    audio = dict(hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=2, head_dim=16, num_mel_bins=8, sliding_window=6)
    cfg = dict(model_type="aero_realtime", backbone_family=family, text_config=text, vision_config=vis, audio_config=audio,
               downsample_factor=2, image_token_index=290, video_token_index=291, audio_token_index=292, vision_start_token_index=293)
    return create_model_from_config("aero_realtime", cfg).eval(), text, vis


def test_generation_with_an_image_prompt_matches_rerunning_the_sequence():
    """Greedy continuation of an image + text prompt on the key / value cache (rotary positions continue after the
    prompt's largest multimodal position) equals re-running the growing sequence through the plain forward pass."""
    from lmms_engine_b200.mapping_func import create_model_from_config
    from lmms_engine_b200.models.generation import generate

    torch.manual_seed(0)
    _, text, vis = _tiny_realtime()
    model = create_model_from_config("qwen3_vl", dict(model_type="qwen3_vl", text_config=text, vision_config=vis, image_token_id=290,
                                                      video_token_id=291, vision_start_token_id=293)).eval()
    ids = torch.randint(0, 280, (30,))
    ids[2], ids[3:7] = 293, 290
    pix, grid = torch.randn(16, 3 * 2 * 4 * 4), torch.tensor([[1, 4, 4]])
    new = generate(model, ids, 6, pixel_values=pix, image_grid_thw=grid)
    seq = ids.clone()
    with torch.no_grad():
        for _ in range(6):
            cu = torch.tensor([0, seq.numel()], dtype=torch.int32)
            hidden = model(input_ids=seq, cu_seqlens=cu, pixel_values=pix, image_grid_thw=grid)["hidden_states"]
            nxt = F.linear(hidden[-1:], model.language_model.lm_head.weight).argmax(-1)
            seq = torch.cat([seq, nxt])
    assert new.tolist() == seq[30:].tolist()
    text_only = create_model_from_config("qwen3", dict(text, model_type="qwen3", rope_scaling=None)).eval()
    a = generate(text_only, ids[:12], 5, temperature=0.8, generator=torch.Generator().manual_seed(1))
    b = generate(text_only, ids[:12], 5, temperature=0.8, generator=torch.Generator().manual_seed(1))
    assert a.tolist() == b.tolist() and a.numel() == 5
    from lmms_engine_b200.models.dllm import DiffusionLM

    masked = create_model_from_config("qwen3_dllm", dict(text, model_type="qwen3_dllm", rope_scaling=None)).eval()
    assert isinstance(masked, DiffusionLM)
    with pytest.raises(NotImplementedError):  # bidirectional masked-token models do not generate left to right
        generate(masked, ids[:12], 2)


def test_realtime_session_streams_slot_by_slot_like_the_full_pass():
    """One audio slot per call: the tokens the session emits are those the full forward pass predicts at the same
    slots when it is given the whole stream at once (chunked audio: every slot is encoded by itself)."""
    from lmms_engine_b200.models.generation import RealtimeSession

    torch.manual_seed(0)
    model, _, _ = _tiny_realtime()
    AS, AE, PAD_TOK = 294, 295, 281
    prompt = torch.cat([torch.randint(0, 280, (10,)), torch.tensor([AS])])
    K = 7
    feats = torch.randn(K, 8, 4)  # one [mel, 2 * downsample_factor] piece per slot
    session = RealtimeSession(model, rt_pad_id=PAD_TOK)
    session.start(prompt)
    first = int(session.last)
    emitted = [session.listen(feats[k]) for k in range(K)]
    ids = torch.cat([prompt, torch.full((K,), 292)])
    stream = torch.cat([prompt, torch.tensor([first] + emitted[:-1])])
    with torch.no_grad():
        cu = torch.tensor([0, ids.numel()], dtype=torch.int32)
        hidden = model(input_ids=ids, cu_seqlens=cu, text_stream_ids=stream, input_features=feats,
                       audio_attention_mask=torch.ones(K, 2, dtype=torch.long))["hidden_states"]
        want = F.linear(hidden, model.language_model.lm_head.weight).argmax(-1)
    assert int(want[10]) == first and want[11:].tolist() == emitted


def test_streaming_audio_encoder_variants_against_plain_torch():
    """LayerNorm + GELU MLP + symmetric convolution padding + attention without causality: the encoder equals a direct
    restatement with library ops; the default stays causal (a change in the last mel frame moves only the last frame)."""
    from lmms_engine_b200.models.audio import VoxtralRealtimeEncoder, VoxtralRealtimeEncoderConfig

    torch.manual_seed(0)
    base = dict(hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=2, head_dim=16, num_mel_bins=8, sliding_window=6)
    c = VoxtralRealtimeEncoderConfig.from_dict(dict(base, norm_type="layer_norm", mlp_type="gelu", conv_padding="symmetric",
                                                    attention_window_left=-1, attention_window_right=-1))
    m = VoxtralRealtimeEncoder(c).eval()
    with torch.no_grad():
        for p in m.parameters():
            p.normal_(0, 0.2)
    x = torch.randn(2, 8, 12)
    sd = m.state_dict()

    def plain(feats):
        h = F.gelu(F.conv1d(F.pad(feats, (1, 1)), sd["embedder.conv1.weight"], sd["embedder.conv1.bias"]))
        h = F.gelu(F.conv1d(F.pad(h, (0, 1)), sd["embedder.conv2.weight"], sd["embedder.conv2.bias"], stride=2)).transpose(1, 2)  # [n, 6, 32]
        n, T, _ = h.shape
        inv = 1.0 / (10000.0 ** (torch.arange(0, 16, 2).float() / 16))
        ang = torch.arange(T).float()[:, None] * inv[None]
        cos, sin = torch.cat([ang.cos(), ang.cos()], -1), torch.cat([ang.sin(), ang.sin()], -1)
        rot = lambda t: torch.cat([-t[..., 8:], t[..., :8]], -1)  # noqa: E731
        for i in range(2):
            pre = f"layers.{i}."
            y = F.layer_norm(h, (32,), sd[pre + "self_attn_layer_norm.weight"], sd[pre + "self_attn_layer_norm.bias"], 1e-5)
            q = F.linear(y, sd[pre + "self_attn.q_proj.weight"], sd[pre + "self_attn.q_proj.bias"]).view(n, T, 2, 16)
            k = F.linear(y, sd[pre + "self_attn.k_proj.weight"]).view(n, T, 2, 16)
            v = F.linear(y, sd[pre + "self_attn.v_proj.weight"], sd[pre + "self_attn.v_proj.bias"]).view(n, T, 2, 16)
            q, k = q * cos[None, :, None] + rot(q) * sin[None, :, None], k * cos[None, :, None] + rot(k) * sin[None, :, None]
            a = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)).transpose(1, 2).reshape(n, T, 32)
            h = h + F.linear(a, sd[pre + "self_attn.o_proj.weight"], sd[pre + "self_attn.o_proj.bias"])
            y = F.layer_norm(h, (32,), sd[pre + "final_layer_norm.weight"], sd[pre + "final_layer_norm.bias"], 1e-5)
            h = h + F.linear(F.gelu(F.linear(y, sd[pre + "mlp.fc1.weight"], sd[pre + "mlp.fc1.bias"])), sd[pre + "mlp.fc2.weight"], sd[pre + "mlp.fc2.bias"])
        return F.layer_norm(h, (32,), sd["norm.weight"], sd["norm.bias"], 1e-5).reshape(n * T, 32)

    with torch.no_grad():
        got = m(x)
        assert got["frame_lengths"].tolist() == [6, 6]
        assert (got["last_hidden_state"] - plain(x)).abs().max() < 2e-5
        causal = VoxtralRealtimeEncoder(VoxtralRealtimeEncoderConfig.from_dict(base)).eval()
        x2 = x.clone()
        x2[:, :, -1] += 1.0
        moved = (causal(x)["last_hidden_state"] - causal(x2)["last_hidden_state"]).abs().reshape(2, 6, -1).amax(-1) > 1e-6
        assert moved.sum(1).tolist() == [1, 1] and moved[:, -1].all()
    with pytest.raises(ValueError):
        VoxtralRealtimeEncoderConfig.from_dict(dict(base, norm_type="batch_norm"))


def test_audio_encoder_stream_equals_the_whole_clip_and_look_ahead_is_bounded():
    """(1) A clip encoded piece by piece on the stream cache (convolution tails, keys / values inside the left window)
    gives the rows of the one-piece pass.  (2) With a look-ahead of two frames, a change in frame j moves frames
    j - 2 ... j + left of a one-layer encoder and nothing else.  (3) The realtime session on continuous audio emits what
    the full pass over the whole clip predicts."""
    from lmms_engine_b200.models.audio import VoxtralRealtimeEncoder, VoxtralRealtimeEncoderConfig
    from lmms_engine_b200.models.generation import RealtimeSession

    torch.manual_seed(0)
    base = dict(hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=2, head_dim=16, num_mel_bins=8, sliding_window=5)
    enc = VoxtralRealtimeEncoder(VoxtralRealtimeEncoderConfig.from_dict(base)).eval()
    with torch.no_grad():
        for p in enc.parameters():
            p.normal_(0, 0.2)
        clip = torch.randn(1, 8, 40)
        whole = enc(clip)["last_hidden_state"]
        cache = enc.new_stream()
        rows = torch.cat([enc.stream(clip[0, :, a:b], cache) for a, b in ((0, 4), (4, 8), (8, 20), (20, 22), (22, 40))])
        assert rows.shape == whole.shape and (rows - whole).abs().max() < 2e-5
        assert cache.frames == 20 and cache.layers[0][0].shape[0] == 4  # sliding_window 5: the frame itself and 4 before it
        with pytest.raises(ValueError):
            enc.stream(clip[0, :, :3], enc.new_stream())

        ahead = VoxtralRealtimeEncoder(VoxtralRealtimeEncoderConfig.from_dict(
            dict(base, num_hidden_layers=1, attention_window_left=3, attention_window_right=2))).eval()
        for p in ahead.parameters():
            p.normal_(0, 0.2)
        with pytest.raises(ValueError):
            ahead.new_stream()
        h = torch.randn(16, 32)
        cu = torch.tensor([0, 16], dtype=torch.int32)
        cos, sin = ahead._rotary(torch.arange(16).float())
        h2 = h.clone()
        h2[9] += 1.0
        layer = ahead.layers[0].self_attn
        moved = ((layer(h, cu, cos, sin) - layer(h2, cu, cos, sin)).abs().amax(-1) > 1e-7).nonzero().flatten().tolist()
        assert moved == list(range(7, 13))  # frame i sees i - 3 ... i + 2, so frame 9 is seen by frames 7 ... 12

    model, _, _ = _tiny_realtime()
    AS, PAD_TOK, K = 294, 281, 6
    prompt = torch.cat([torch.randint(0, 280, (10,)), torch.tensor([AS])])
    feats = torch.randn(8, 4 * K)
    session = RealtimeSession(model, rt_pad_id=PAD_TOK, continuous_audio=True)
    session.start(prompt)
    first = int(session.last)
    emitted = [session.listen(feats[:, 4 * k:4 * k + 4]) for k in range(K)]
    ids = torch.cat([prompt, torch.full((K,), 292)])
    stream = torch.cat([prompt, torch.tensor([first] + emitted[:-1])])
    with torch.no_grad():
        cu = torch.tensor([0, ids.numel()], dtype=torch.int32)
        hidden = model(input_ids=ids, cu_seqlens=cu, text_stream_ids=stream, input_features=feats[None],
                       audio_attention_mask=torch.ones(1, 2 * K, dtype=torch.long))["hidden_states"]
        want = F.linear(hidden, model.language_model.lm_head.weight).argmax(-1)
    assert int(want[10]) == first and want[11:].tolist() == emitted
