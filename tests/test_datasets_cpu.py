"""Data plane on CPU: packers, processors, map-style and iterable datasets, collators."""
import json
import os
import random
import sys

import numpy as np
import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


@pytest.mark.parametrize("name", ["first_fit", "best_fit", "balanced", "true_first_fit"])
def test_online_packers_lose_nothing_and_respect_budget(name):
    from lmms_engine_b200.datasets.packing import build_online_packer

    rng = random.Random(1)
    packer = build_online_packer(name, 2048)
    lens = [rng.randint(1, 2048) for _ in range(2000)]
    seen = []
    for i, n in enumerate(lens):
        for pack in packer.add((i, n), n):
            assert sum(x[1] for x in pack) <= 2048
            seen += [x[0] for x in pack]
    for pack in packer.flush():
        assert sum(x[1] for x in pack) <= 2048
        seen += [x[0] for x in pack]
    assert sorted(seen) == list(range(2000))


def test_first_fit_is_next_fit_like_the_reference():
    from lmms_engine_b200.datasets.packing import FirstFitPacking, pack_by_first_fit, pack_by_window

    p = FirstFitPacking(10)
    out = []
    for i, n in enumerate([6, 3, 4, 5, 5, 1]):
        out += list(p.add(i, n))
    out += list(p.flush())
    assert out == [[0, 1], [2, 3], [4, 5]]  # the open pack is never revisited
    assert pack_by_first_fit([6, 3, 4, 5, 5, 1], 10) == [[0, 1], [2, 3], [4, 5]]
    groups = pack_by_window([6, 3, 4, 5, 5, 1], 10, 6)
    assert sorted(i for g in groups for i in g) == list(range(6))
    assert all(sum([6, 3, 4, 5, 5, 1][i] for i in g) <= 10 for g in groups)


def test_best_fit_packs_tighter_than_next_fit():
    from lmms_engine_b200.datasets.packing import build_online_packer

    rng = random.Random(3)
    lens = [rng.randint(100, 1500) for _ in range(3000)]

    def n_packs(name):
        p = build_online_packer(name, 4096)
        k = 0
        for i, n in enumerate(lens):
            k += len(list(p.add(i, n)))
        return k + len(list(p.flush()))

    assert n_packs("best_fit") <= n_packs("first_fit")
    assert n_packs("balanced") <= n_packs("first_fit")


def _write_records(path, n=40):
    recs = []
    for i in range(n):
        recs.append({"id": i, "messages": [
            {"role": "user", "content": [{"type": "text", "text": "question " * (1 + i % 7)}]},
            {"role": "assistant", "content": [{"type": "text", "text": f"answer {i}"}]}]})
    with open(path, "w") as f:
        for r in recs:
            f.write(json.dumps(r) + "\n")
    return recs


def test_labels_supervise_assistant_only(tmp_path):
    from lmms_engine_b200.datasets.config import ProcessorConfig
    from lmms_engine_b200.datasets.processor import ChatProcessor

    p = ChatProcessor(ProcessorConfig(processor_name="byte", processor_type="qwen2")).build()
    out = p.process([{"role": "user", "content": [{"type": "text", "text": "hi"}]},
                     {"role": "assistant", "content": [{"type": "text", "text": "hello"}]}])
    sup = out["input_ids"][out["labels"] != -100]
    assert p.tokenizer.decode(sup) == "hello<|im_end|>\n"
    assert (out["labels"][out["labels"] != -100] == sup).all()


def test_iterable_dataset_packs_shards_and_resumes(tmp_path):
    from lmms_engine_b200.datasets.config import DatasetConfig
    from lmms_engine_b200.datasets import registry  # noqa: F401
    from lmms_engine_b200.mapping_func import DATASET_MAPPING

    path = tmp_path / "d.jsonl"
    _write_records(path)
    cfg = DatasetConfig(dataset_type="vision_iterable", dataset_format="jsonl", dataset_path=str(path),
                        processor_config={"processor_name": "byte", "processor_type": "qwen2"}, packing=True,
                        packing_strategy="first_fit", packing_length=512, shuffle=True, data_seed=3)
    ds = DATASET_MAPPING["vision_iterable"](cfg).build()
    packs = list(ds)
    assert sum(len(p) for p in packs) == 40
    assert all(sum(s["input_ids"].numel() for s in p) <= 512 for p in packs)
    # resume after two packs reproduces the tail exactly
    ds2 = DATASET_MAPPING["vision_iterable"](cfg).build()
    it = iter(ds2)
    next(it); next(it)
    state = ds2.state_dict()
    ds3 = DATASET_MAPPING["vision_iterable"](cfg).build()
    ds3.load_state_dict(state)
    tail = list(ds3)
    assert [[s["input_ids"].tolist() for s in p] for p in tail] == [[s["input_ids"].tolist() for s in p] for p in packs[2:]]
    batch = ds.get_collator()([packs[0]])
    assert batch["input_ids"].dim() == 1 and batch["cu_seqlens"][-1] == batch["input_ids"].numel()
    assert batch["position_ids"][batch["cu_seqlens"][1]] == 0


def test_iterable_dataset_second_epoch_and_oversize_order(tmp_path):
    """A second pass over the dataset (num_workers=0) yields the same packs as the first; a sample longer
    than the packing length comes out alone, after whatever the packer held before it."""
    from lmms_engine_b200.datasets.config import DatasetConfig
    from lmms_engine_b200.datasets import registry  # noqa: F401
    from lmms_engine_b200.mapping_func import DATASET_MAPPING

    path = tmp_path / "d.jsonl"
    _write_records(path)
    cfg = DatasetConfig(dataset_type="vision_iterable", dataset_format="jsonl", dataset_path=str(path),
                        processor_config={"processor_name": "byte", "processor_type": "qwen2"}, packing=True,
                        packing_strategy="first_fit", packing_length=512, shuffle=False)
    ds = DATASET_MAPPING["vision_iterable"](cfg).build()
    first = [[s["input_ids"].tolist() for s in p] for p in ds]
    second = [[s["input_ids"].tolist() for s in p] for p in ds]
    assert len(first) > 0 and first == second
    # a resumed pass continues from the cursor, the pass after it starts over
    ds.load_state_dict({"cur_idx": 30})
    assert sum(len(p) for p in ds) == 10
    assert sum(len(p) for p in ds) == 40
    # oversize: with a packing length below the longest record, stream order is preserved
    lens = [int(s["input_ids"].numel()) for p in DATASET_MAPPING["vision_iterable"](cfg).build() for s in p]
    cut = sorted(lens)[len(lens) // 2]
    cfg2 = DatasetConfig(dataset_type="vision_iterable", dataset_format="jsonl", dataset_path=str(path),
                         processor_config={"processor_name": "byte", "processor_type": "qwen2"}, packing=True,
                         packing_strategy="first_fit", packing_length=cut, shuffle=False, filter_overlong=False)
    ds2 = DATASET_MAPPING["vision_iterable"](cfg2).build()
    out = [int(s["input_ids"].numel()) for p in ds2 for s in p]
    assert out == lens
    assert any(len(p) == 1 and p[0]["input_ids"].numel() > cut for p in ds2)
    # ranks share every record: 40 records over 3 ranks -> 14 + 13 + 13
    sizes = []
    for r in range(3):
        d = DATASET_MAPPING["vision_iterable"](cfg).build()
        d.dp_rank, d.dp_size = r, 3
        sizes.append(sum(len(p) for p in d))
    assert sizes == [14, 13, 13]


def test_map_dataset_offline_packing_and_padded_collator(tmp_path):
    from lmms_engine_b200.datasets.config import DatasetConfig
    from lmms_engine_b200.datasets import registry  # noqa: F401
    from lmms_engine_b200.mapping_func import DATASET_MAPPING

    path = tmp_path / "d.jsonl"
    _write_records(path)
    cfg = DatasetConfig(dataset_type="vision", dataset_format="jsonl", dataset_path=str(path),
                        processor_config={"processor_name": "byte", "processor_type": "qwen2"}, packing=True,
                        packing_strategy="window_8", packing_length=64, extra_kwargs={"collator_type": "vision"})
    ds = DATASET_MAPPING["vision"](cfg).build()
    assert sorted(i for g in ds.groups for i in g) == list(range(40))
    assert len(ds.modality_length) == len(ds) and all(n < 0 for n in ds.modality_length)
    batch = ds.get_collator()([ds[0]])
    assert batch["input_ids"].dim() == 2 and batch["attention_mask"].shape == batch["input_ids"].shape
    assert (batch["labels"][batch["attention_mask"] == 0] == -100).all()


def test_vl_processor_counts_and_patch_order():
    from lmms_engine_b200.datasets.config import ProcessorConfig
    from lmms_engine_b200.datasets.processor import QwenVLProcessor
    from lmms_engine_b200.datasets.processor import vision_process as vp

    assert vp.smart_resize(100, 150, 28) == (112, 140)
    h, w = vp.smart_resize(4000, 3000, 28, max_pixels=1280 * 28 * 28)
    assert h % 28 == 0 and w % 28 == 0 and h * w <= 1280 * 28 * 28
    p = QwenVLProcessor(ProcessorConfig(processor_name="byte", processor_type="qwen2_5_vl")).build()
    img = (np.random.rand(100, 150, 3) * 255).astype(np.uint8)
    out = p.process([{"role": "user", "content": [{"type": "image", "image": "x"}, {"type": "text", "text": "?"}]},
                     {"role": "assistant", "content": [{"type": "text", "text": "ok"}]}], images=[img])
    t, gh, gw = out["image_grid_thw"][0].tolist()
    assert (out["input_ids"] == p.image_token_id).sum().item() == t * gh * gw // 4
    assert out["pixel_values"].shape == (t * gh * gw, 3 * 2 * 14 * 14)
    assert out["position_ids"].shape == (3, out["input_ids"].numel())
    # first patch row = top-left 14x14 patch, channel-major, both temporal copies
    arr = np.asarray(__import__("PIL.Image", fromlist=["Image"]).fromarray(img).resize((140, 112), 3)).astype(np.float32) / 255
    ref = ((arr[:14, :14] - np.array(vp.CLIP_MEAN)) / np.array(vp.CLIP_STD)).transpose(2, 0, 1)
    got = out["pixel_values"][0].view(3, 2, 14, 14)
    assert torch.allclose(got[:, 0], torch.from_numpy(ref).float(), atol=1e-5)
    # second row of the stream is the patch to the right inside the same 2x2 block
    ref2 = ((arr[:14, 14:28] - np.array(vp.CLIP_MEAN)) / np.array(vp.CLIP_STD)).transpose(2, 0, 1)
    assert torch.allclose(out["pixel_values"][1].view(3, 2, 14, 14)[:, 0], torch.from_numpy(ref2).float(), atol=1e-5)


def test_extra_datasets_and_processors(tmp_path):
    """fineweb_edu text rows pack with every token supervised; sit / rae rows become tensors; the
    nanovlm processor emits one placeholder per NaFlex patch."""
    import json

    import numpy as np
    from PIL import Image

    from lmms_engine_b200.datasets import registry  # noqa: F401
    from lmms_engine_b200.datasets.config import DatasetConfig
    from lmms_engine_b200.mapping_func import DATAPROCESSOR_MAPPING, DATASET_MAPPING

    for name in ("fineweb_edu", "sit", "rae", "vision", "vision_iterable", "qwen3_vl_iterable"):
        assert name in DATASET_MAPPING, name
    for name in ("sit", "rae_siglip", "wanvideo", "nanovlm", "pure_text", "qwen2_5_vl", "qwen3_vl"):
        assert name in DATAPROCESSOR_MAPPING, name
    txt = tmp_path / "t.jsonl"
    txt.write_text("\n".join(json.dumps({"text": "hello world " * (5 + i)}) for i in range(12)))
    ds = DATASET_MAPPING["fineweb_edu"](DatasetConfig(dataset_type="fineweb_edu", dataset_format="jsonl", dataset_path=str(txt),
                                                      processor_config={"processor_name": "none", "processor_type": "pure_text"},
                                                      packing=True, packing_length=256, shuffle=False)).build()
    packs = list(ds)
    assert packs and all(sum(s["input_ids"].numel() for s in p) <= 256 for p in packs)
    assert sum(len(p) for p in packs) == 12 and all(torch.equal(s["input_ids"], s["labels"]) for p in packs for s in p)
    # sit / rae
    np.save(tmp_path / "lat.npy", np.random.randn(4, 8, 8).astype("float32"))
    Image.fromarray((np.random.rand(40, 60, 3) * 255).astype("uint8")).save(tmp_path / "im.png")
    (tmp_path / "sit.json").write_text(json.dumps([{"latent": str(tmp_path / "lat.npy"), "label": 3}] * 2))
    (tmp_path / "rae.json").write_text(json.dumps([{"image": str(tmp_path / "im.png")}] * 2))
    sit = DATASET_MAPPING["sit"](DatasetConfig(dataset_type="sit", dataset_format="json", dataset_path=str(tmp_path / "sit.json"),
                                               processor_config={"processor_name": "none", "processor_type": "sit"})).build()
    b = sit.get_collator()([sit[0], sit[1]])
    assert b["latents"].shape == (2, 4, 8, 8) and b["labels"].tolist() == [3, 3]
    rae = DATASET_MAPPING["rae"](DatasetConfig(dataset_type="rae", dataset_format="json", dataset_path=str(tmp_path / "rae.json"),
                                               processor_config={"processor_name": "none", "processor_type": "rae_siglip",
                                                                 "extra_kwargs": {"image_size": 32}})).build()
    assert rae[0]["pixel_values"].shape == (3, 32, 32) and rae[0]["pixel_values"].abs().max() <= 1.0 + 1e-6
    # nanovlm processor
    from lmms_engine_b200.datasets.config import ProcessorConfig

    proc = DATAPROCESSOR_MAPPING["nanovlm"](ProcessorConfig(processor_name="none", processor_type="nanovlm",
                                                            extra_kwargs={"patch_size": 8, "max_num_patches": 24})).build()
    msgs = [{"role": "user", "content": [{"type": "image"}, {"type": "text", "text": "what"}]},
            {"role": "assistant", "content": [{"type": "text", "text": "a picture"}]}]
    out = proc.process(msgs, images=[Image.open(tmp_path / "im.png")])
    rows, cols = out["spatial_shapes"][0].tolist()
    assert rows * cols <= 24 and out["pixel_values"].shape == (rows * cols, 3 * 64)
    assert int((out["input_ids"] == proc.image_token_id).sum()) == rows * cols


def test_log_mel_matches_whisper_extractor_and_audio_processor_counts():
    import numpy as np

    from lmms_engine_b200.datasets import registry  # noqa: F401
    from lmms_engine_b200.datasets.config import ProcessorConfig
    from lmms_engine_b200.datasets.processor.audio_process import log_mel_spectrogram
    from lmms_engine_b200.mapping_func import DATAPROCESSOR_MAPPING

    wav = (np.sin(2 * np.pi * 440 * np.arange(16000 * 2) / 16000) * 0.5).astype("float32")
    feats, mask, valid = log_mel_spectrogram(wav, 128, 3000)
    assert feats.shape == (128, 3000) and valid == 200 and int(mask.sum()) == 200
    try:
        from transformers import WhisperFeatureExtractor

        ref = WhisperFeatureExtractor(feature_size=128)(wav, sampling_rate=16000, return_tensors="pt")["input_features"][0]
        assert (ref - feats).abs().max() < 1e-4
    except ImportError:
        pass
    proc = DATAPROCESSOR_MAPPING["qwen2_audio"](ProcessorConfig(processor_name="none", processor_type="qwen2_audio")).build()
    msgs = [{"role": "user", "content": [{"type": "audio"}, {"type": "text", "text": "what is this"}]},
            {"role": "assistant", "content": [{"type": "text", "text": "a tone"}]}]
    out = proc.process(msgs, audios=[wav])
    assert out["audio_values"].shape == (1, 128, 3000)
    assert int((out["input_ids"] == proc.audio_token_id).sum()) == 50  # 200 mel frames -> 100 -> 50 pooled rows
    assert (out["labels"][out["input_ids"] == proc.audio_token_id] == -100).all()


def test_bagel_dataset_processor_collator_feed_the_model(tmp_path):
    """Interleaved text / image conversations -> packed stream with latent tokens -> one training step of the model."""
    import numpy as np
    from PIL import Image

    from lmms_engine_b200.datasets import registry  # noqa: F401
    from lmms_engine_b200.datasets.config import DatasetConfig
    from lmms_engine_b200.mapping_func import DATASET_MAPPING, create_model_from_config

    torch.manual_seed(0)
    torch.save(torch.randn(3, 8, 12), tmp_path / "gen.pt")
    np.save(tmp_path / "cond.npy", np.random.randn(3, 4, 4).astype(np.float32))
    Image.fromarray((np.random.rand(40, 64, 3) * 255).astype(np.uint8)).save(tmp_path / "photo.png")
    records = [
        {"messages": [{"role": "user", "content": [{"type": "text", "text": "draw a cat"}]},
                      {"role": "assistant", "content": [{"type": "image_url", "image_url": {"url": "gen.pt"}}]}]},
        {"messages": [{"role": "user", "content": [{"type": "image_url", "image_url": {"url": "cond.npy"}},
                                                   {"type": "text", "text": "what is it"}]},
                      {"role": "assistant", "content": [{"type": "text", "text": "a dog"}]}]},
        {"messages": [{"role": "user", "content": [{"type": "image_url", "image_url": {"url": "photo.png"}},
                                                   {"type": "text", "text": "same, at night"}]},
                      {"role": "assistant", "content": [{"type": "image_url", "image_url": {"url": "gen.pt"}}]}]},
    ]
    path = tmp_path / "d.jsonl"
    path.write_text("".join(json.dumps(r) + "\n" for r in records))
    cfg = DatasetConfig(dataset_type="bagel_iterable", dataset_format="jsonl", dataset_path=str(path), shuffle=False, packing=False,
                        processor_config={"processor_name": "byte", "processor_type": "bagel",
                                          "extra_kwargs": {"latent_patch_size": 2, "vae_downsample": 8, "max_latent_size": 8,
                                                           "latent_from_pixels": True}},
                        extra_kwargs={"data_folder": str(tmp_path)})
    ds = DATASET_MAPPING["bagel_iterable"](cfg).build()
    ds.data_folder = [str(tmp_path)] * len(ds.data_list)
    samples = [s for pack in ds for s in pack]
    assert len(samples) == 3
    a, b, c = samples
    p = ds.processor
    # generation target: 4 x 6 tokens of 3*2*2 values between the vision markers, one rotary position, noise level in (0, 1)
    assert a["latent_tokens"].shape == (24, 12) and a["latent_loss_mask"].all() and 0 < float(a["timesteps"][0]) < 1
    start = int(a["latent_index"][0])
    assert a["input_ids"][start - 1] == p.vision_start and a["input_ids"][start + 24] == p.vision_end
    assert a["position_ids"][start - 1] == a["position_ids"][start + 24] and (a["labels"] == -100).all()
    assert a["latent_pos"][:7].tolist() == [0, 1, 2, 3, 4, 5, 8]
    # understanding: clean condition image, assistant text supervised (own tokens, the model shifts)
    assert not b["latent_loss_mask"].any() and float(b["timesteps"].max()) == 0.0
    sup = b["labels"] != -100
    assert p.tokenizer.decode(b["input_ids"][sup].tolist()) == "a dog<|im_end|>"
    assert c["latent_tokens"].shape[0] == (40 // 16) * (64 // 16) + 24  # pooled photo + target
    batch = ds.get_collator()([samples])
    assert batch["cu_seqlens"].tolist() == [0, a["input_ids"].numel(), a["input_ids"].numel() + b["input_ids"].numel(),
                                            sum(s["input_ids"].numel() for s in samples)]
    assert int(batch["latent_index"][24]) == a["input_ids"].numel() + int(b["latent_index"][0])
    model = create_model_from_config("bagel", dict(model_type="bagel", vocab_size=p.tokenizer.vocab_size + 64, hidden_size=32,
                                                   intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
                                                   num_key_value_heads=2, latent_channels=3, latent_patch_size=2, max_latent_size=8))
    out = model(**batch)
    out["loss"].backward()
    assert torch.isfinite(out["loss"]) and out["ce"] is not None and out["mse"] is not None


def test_aero_realtime_processor_places_speech_on_the_audio_timeline(tmp_path):
    """One slot per 80 ms; silence supervised as rt_pad, a speech segment written after its start time with an
    unsupervised context slot; the collated batch drives the model."""
    import numpy as np

    from lmms_engine_b200.datasets import registry  # noqa: F401
    from lmms_engine_b200.datasets.config import ProcessorConfig
    from lmms_engine_b200.mapping_func import DATAPROCESSOR_MAPPING, DATASET_MAPPING, create_model_from_config

    proc = DATAPROCESSOR_MAPPING["aero_realtime"](ProcessorConfig(processor_name="byte_realtime", processor_type="aero_realtime",
                                                                   extra_kwargs={"num_mel_bins": 16, "downsample_factor": 4})).build()
    wave = np.random.default_rng(0).standard_normal(16000 * 2).astype(np.float32)  # 2 s -> 200 mel frames -> 100 frames -> 25 slots
    msgs = [{"role": "user", "content": [{"type": "audio", "audio": "clip"}]}]
    segs = [{"role": "assistant", "time": 0.5, "text": "hi!"}, {"role": "user", "time": 0.1, "text": "ignored"}]
    out = proc.process(msgs, audios=[wave], realtime_segments=segs)
    ids, stream, labels = out["input_ids"], out["text_stream_ids"], out["labels"]
    slots = torch.nonzero(ids == proc.audio_token_id).flatten()
    assert slots.numel() == 25 and ids[slots[0] - 1] == proc.audio_start and ids[slots[-1] + 1] == proc.audio_end
    assert out["input_features"].shape == (1, 16, 200) and int(out["feature_attention_mask"].sum()) == 200
    first = 7  # 0.5 s / 0.08 s -> slot 7 (0.56 s) is the first at or after the start time
    assert abs(proc.seconds_per_slot - 0.08) < 1e-9
    assert stream[slots[first]] == proc.rt_pad and labels[slots[first]] == -100
    said = stream[slots[first + 1:first + 4]].tolist()
    assert bytes(said).decode() == "hi!" and labels[slots[first + 1:first + 4]].tolist() == said
    others = [k for k in range(25) if not first <= k <= first + 3]
    assert all(stream[slots[k]] == proc.rt_pad and labels[slots[k]] == proc.rt_pad for k in others)
    assert torch.equal(stream[ids != proc.audio_token_id], ids[ids != proc.audio_token_id])
    # dataset + collator + model
    import wave as wavelib

    from lmms_engine_b200.datasets.config import DatasetConfig

    for name, seconds in (("a.wav", 1.0), ("b.wav", 0.5)):
        with wavelib.open(str(tmp_path / name), "wb") as w:
            w.setnchannels(1), w.setsampwidth(2), w.setframerate(16000)
            w.writeframes((np.random.default_rng(1).standard_normal(int(16000 * seconds)) * 3000).astype(np.int16).tobytes())
    records = [{"messages": [{"role": "user", "content": [{"type": "audio_url", "audio_url": {"url": "a.wav"}}]}],
                "realtime_segments": [{"role": "assistant", "time": 0.2, "text": "ok"}]},
               {"messages": [{"role": "user", "content": [{"type": "audio_url", "audio_url": {"url": "b.wav"}},
                                                          {"type": "text", "text": "what was said"}]},
                             {"role": "assistant", "content": [{"type": "text", "text": "nothing"}]}]}]
    path = tmp_path / "rt.jsonl"
    path.write_text("".join(json.dumps(r) + "\n" for r in records))
    cfg = DatasetConfig(dataset_type="aero_realtime_iterable", dataset_format="jsonl", dataset_path=str(path), shuffle=False,
                        packing=False, processor_config={"processor_name": "byte_realtime", "processor_type": "aero_realtime",
                                                         "extra_kwargs": {"num_mel_bins": 16, "downsample_factor": 4}})
    ds = DATASET_MAPPING["aero_realtime_iterable"](cfg).build()
    ds.data_folder = [str(tmp_path)] * len(ds.data_list)
    samples = [s for pack in ds for s in pack]
    assert [int((s["input_ids"] == proc.audio_token_id).sum()) for s in samples] == [12, 6]
    batch = ds.get_collator()([samples])
    assert batch["input_features"].shape == (2, 16, 100) and batch["text_stream_ids"].shape == batch["input_ids"].shape
    text = dict(vocab_size=len(proc.tokenizer) + 6, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
                num_key_value_heads=2, head_dim=8, rope_scaling={"mrope_section": [2, 1, 1], "mrope_interleaved": True})
    vis = dict(depth=1, hidden_size=16, intermediate_size=32, num_heads=2, patch_size=4, out_hidden_size=32, num_position_embeddings=16,
               deepstack_visual_indexes=[])
    audio = dict(hidden_size=16, intermediate_size=32, num_hidden_layers=1, num_attention_heads=2, head_dim=8, num_mel_bins=16, sliding_window=8)
    model = create_model_from_config("aero_realtime", dict(model_type="aero_realtime", backbone_family="qwen3_vl", text_config=text,
                                                           vision_config=vis, audio_config=audio, downsample_factor=4,
                                                           audio_token_index=proc.audio_token_id))
    loss = model(**batch)["loss"]
    loss.backward()
    assert torch.isfinite(loss) and model.multi_modal_projector.linear_1.weight.grad.abs().sum() > 0


def _realtime_processor(**extra):
    from lmms_engine_b200.datasets import registry  # noqa: F401
    from lmms_engine_b200.datasets.config import ProcessorConfig
    from lmms_engine_b200.mapping_func import DATAPROCESSOR_MAPPING

    kw = {"num_mel_bins": 16, "downsample_factor": 4, "patch_size": 4, "min_pixels": 64, "max_pixels": 256}
    kw.update(extra)
    return DATAPROCESSOR_MAPPING["aero_realtime"](ProcessorConfig(processor_name="byte_realtime", processor_type="aero_realtime",
                                                                   extra_kwargs=kw)).build()


def test_aero_realtime_interleaves_video_chunks_with_their_audio_slots():
    """A 2 s video of 8 frames at 4 fps with its 2 s track: 4 temporal patches stamped 0.1 / 0.6 / 1.1 / 1.6 s; the 25
    slots of 80 ms are split at those stamps; typed text goes in front of the first patch at or after its time; speech
    goes into the slots from its start time on, across envelope boundaries."""
    from lmms_engine_b200.datasets.realtime import split_slots_over_chunks

    assert split_slots_over_chunks(25, [0.125, 0.625, 1.125, 1.625], 12.5) == [8, 7, 6, 4]
    assert split_slots_over_chunks(3, [], 12.5) == [] and split_slots_over_chunks(0, [0.0, 1.0], 12.5) == [0, 0]
    proc = _realtime_processor()
    frames = np.random.default_rng(0).integers(0, 255, (8, 16, 16, 3)).astype(np.uint8)
    wave = np.random.default_rng(1).standard_normal(32000).astype(np.float32)
    meta = [{"fps": 4.0, "frames_indices": list(range(8))}]
    msgs = [{"role": "user", "content": [{"type": "video", "video": "clip.mp4"}]}]
    segs = [{"role": "assistant", "time": 0.5, "text": "a cat walks by"}, {"role": "user", "time": 1.0, "text": "what now?"}]
    out = proc.process(msgs, videos=[frames], audios=[wave], realtime_segments=segs, video_metadata=meta)
    ids, stream, labels = out["input_ids"].tolist(), out["text_stream_ids"].tolist(), out["labels"].tolist()
    t, h, w = out["video_grid_thw"][0].tolist()
    assert t == 4 and out["pixel_values_videos"].shape[0] == t * h * w
    per_patch = h * w // 4
    starts = [i for i, x in enumerate(ids) if x == proc.audio_start]
    ends = [i for i, x in enumerate(ids) if x == proc.audio_end]
    assert [e - s - 1 for s, e in zip(starts, ends)] == [8, 7, 6, 4]
    text = proc.tokenizer.decode(ids)
    for stamp in ("<0.1 seconds>", "<0.6 seconds>", "<1.1 seconds>", "<1.6 seconds>"):
        assert stamp in text
    assert text.index("what now?") < text.index("<1.1 seconds>") and text.index("what now?") > text.index("<0.6 seconds>")
    for s in starts:  # every audio envelope directly follows its video envelope
        assert ids[s - 1] == proc.vision_end and ids[s - 1 - per_patch:s - 1] == [proc.video_token_id] * per_patch
    slots = [i for i, x in enumerate(ids) if x == proc.audio_token_id]
    assert len(slots) == 25 and out["input_features"].shape == (1, 16, 200)
    # slots carry their patch's stamp: the first slot at or after 0.5 s is the first of the second envelope (index 8)
    said = list(b"a cat walks by")
    assert stream[slots[8]] == proc.rt_pad and labels[slots[8]] == -100
    assert [stream[slots[k]] for k in range(9, 9 + len(said))] == said == [labels[slots[k]] for k in range(9, 9 + len(said))]
    quiet = [k for k in range(25) if not 8 <= k < 9 + len(said)]
    assert all(stream[slots[k]] == proc.rt_pad == labels[slots[k]] for k in quiet)
    off = [i for i in range(len(ids)) if i not in slots]
    assert all(labels[i] == -100 and stream[i] == ids[i] for i in off)
    assert out["position_ids"].shape == (3, len(ids))


def test_aero_realtime_answers_questions_in_silent_slots_after_the_video():
    """Without timed segments a (question, answer) pair becomes ``question <audio_start> pad x n <audio_end>`` inside
    the user turn: the stream carries the answer, the labels supervise it, and n slots of silence join the features;
    the sample runs through the model in both audio layouts."""
    from lmms_engine_b200.datasets.realtime import RealtimeCollator
    from lmms_engine_b200.mapping_func import create_model_from_config

    frames = np.random.default_rng(0).integers(0, 255, (4, 16, 16, 3)).astype(np.uint8)
    wave = np.random.default_rng(1).standard_normal(16000).astype(np.float32)
    msgs = [{"role": "user", "content": [{"type": "video", "video": "clip.mp4"}, {"type": "text", "text": "what is it?"}]},
            {"role": "assistant", "content": [{"type": "text", "text": "a cat"}]}]
    for chunked in (False, True):
        proc = _realtime_processor(chunk_audio=chunked)
        out = proc.process(msgs, videos=[frames], audios=[wave], video_fps=[4.0])
        ids, stream, labels = out["input_ids"].tolist(), out["text_stream_ids"].tolist(), out["labels"].tolist()
        answer, n_track = list(b"a cat"), 12  # 1 s -> 100 mel frames -> 12 slots
        slots = [i for i, x in enumerate(ids) if x == proc.audio_token_id]
        assert len(slots) == n_track + len(answer)
        tail = slots[n_track:]
        assert [stream[i] for i in tail] == answer == [labels[i] for i in tail]
        assert ids[tail[0] - 1] == proc.audio_start and ids[tail[-1] + 1] == proc.audio_end
        question = list(b"what is it?")
        assert ids[tail[0] - 1 - len(question):tail[0] - 1] == question
        assert ids[-2] == proc.im_end and sum(1 for x in ids if x == proc.im_end) == 2  # system + the one user turn
        assert all(labels[i] == proc.rt_pad for i in slots[:n_track])
        if chunked:
            assert out["input_features"].shape == (n_track + len(answer), 16, 8)
            assert out["feature_attention_mask"].shape == (n_track + len(answer), 4)
            assert float(out["input_features"][n_track:].abs().sum()) == 0.0
        else:
            assert out["input_features"].shape == (2, 16, 100) and out["feature_attention_mask"].sum(-1).tolist() == [100, 40]
        batch = RealtimeCollator()([[out]])
        text = dict(vocab_size=len(proc.tokenizer) + 6, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
                    num_key_value_heads=2, head_dim=8, rope_scaling={"mrope_section": [2, 1, 1], "mrope_interleaved": True})
        vis = dict(depth=1, hidden_size=16, intermediate_size=32, num_heads=2, patch_size=4, out_hidden_size=32,
                   num_position_embeddings=16, deepstack_visual_indexes=[])
        audio = dict(hidden_size=16, intermediate_size=32, num_hidden_layers=1, num_attention_heads=2, head_dim=8, num_mel_bins=16,
                     sliding_window=8)
        model = create_model_from_config("aero_realtime", dict(
            model_type="aero_realtime", backbone_family="qwen3_vl", text_config=text, vision_config=vis, audio_config=audio,
            downsample_factor=4, audio_token_index=proc.audio_token_id, video_token_id=proc.video_token_id,
            image_token_id=proc.image_token_id, vision_start_token_id=proc.vision_start))
        rows = model.audio_rows(batch["input_features"].float(), batch["feature_attention_mask"])
        assert rows.shape[0] == len(slots)
        loss = model(**batch)["loss"]
        loss.backward()
        assert torch.isfinite(loss) and model.visual.patch_embed.proj.weight.grad is not None


def test_aero_realtime_dataset_reads_timed_messages_and_the_sound_track(tmp_path):
    """``"realtime": true`` records: messages with a ``time`` become segments, the video brings the ``.wav`` next to it,
    ``user_audio`` is mixed onto it."""
    from lmms_engine_b200.datasets import registry  # noqa: F401
    from lmms_engine_b200.datasets.config import DatasetConfig
    from lmms_engine_b200.datasets.realtime import mix_onto_track
    from lmms_engine_b200.mapping_func import DATASET_MAPPING

    mixed = mix_onto_track(np.zeros(10, np.float32), np.ones(4, np.float32) * 0.5, 0.5, 16)
    assert mixed.shape == (12,) and mixed[8:].tolist() == [0.5] * 4 and float(mixed[:8].sum()) == 0.0
    _write_video(tmp_path / "v.mp4", n_frames=16, fps=8.0)
    _write_wav(tmp_path / "v.wav", 2.0)
    _write_wav(tmp_path / "q.wav", 0.25)
    record = {"realtime": True, "user_audio": [{"path": "q.wav", "start_time": 0.5}],
              "messages": [{"role": "user", "content": [{"type": "video_url", "video_url": {"url": "v.mp4"}}]},
                           {"role": "user", "time": 0.4, "content": [{"type": "text", "text": "tell me"}]},
                           {"role": "assistant", "time": 1.0, "content": [{"type": "text", "text": "ok"}]}]}
    path = tmp_path / "rt.jsonl"
    path.write_text(json.dumps(record) + "\n")
    cfg = DatasetConfig(dataset_type="aero_realtime_iterable", dataset_format="jsonl", dataset_path=str(path), shuffle=False,
                        packing=False, fps=4, processor_config={"processor_name": "byte_realtime", "processor_type": "aero_realtime",
                                                                 "extra_kwargs": {"num_mel_bins": 16, "patch_size": 4, "min_pixels": 64,
                                                                                  "max_pixels": 256}})
    ds = DATASET_MAPPING["aero_realtime_iterable"](cfg).build()
    ds.data_folder = [str(tmp_path)] * len(ds.data_list)
    (sample,) = [s for pack in ds for s in pack]
    proc = ds.processor
    ids, stream, labels = sample["input_ids"], sample["text_stream_ids"], sample["labels"]
    text = proc.tokenizer.decode(ids.tolist())
    assert "tell me" in text and "ok" not in text.replace("tokens", "")
    slots = torch.nonzero(ids == proc.audio_token_id).flatten()
    assert slots.numel() == 25
    spoken = [i for i in slots.tolist() if labels[i] not in (-100, proc.rt_pad)]
    assert bytes(stream[spoken].tolist()) == b"ok" and labels[spoken].tolist() == stream[spoken].tolist()
    assert int((ids == proc.audio_start).sum()) == int(sample["video_grid_thw"][0, 0])


# ------------------------------------------------------------------------------------------------
# datasets with record handling of their own (datasets/families.py)
def _write_video(path, n_frames=24, fps=8.0, size=(64, 64)):
    import cv2

    wr = cv2.VideoWriter(str(path), cv2.VideoWriter_fourcc(*"mp4v"), fps, size)
    assert wr.isOpened()
    rng = np.random.default_rng(0)
    for i in range(n_frames):
        wr.write((rng.integers(0, 255, (size[1], size[0], 3)) * 0 + (i * 10) % 255).astype(np.uint8))
    wr.release()


def _write_wav(path, seconds, sr=16000):
    import wave as wavelib

    data = (np.sin(np.arange(int(seconds * sr)) * 0.05) * 8000).astype(np.int16)
    with wavelib.open(str(path), "wb") as w:
        w.setnchannels(1), w.setsampwidth(2), w.setframerate(sr)
        w.writeframes(data.tobytes())


def _family_dataset(tmp_path, name, processor_type, records, **cfg):
    from lmms_engine_b200.datasets import registry  # noqa: F401
    from lmms_engine_b200.datasets.config import DatasetConfig
    from lmms_engine_b200.mapping_func import DATASET_MAPPING

    path = tmp_path / f"{name}.jsonl"
    with open(path, "w") as f:
        for r in records:
            f.write(json.dumps(r) + "\n")
    extra = cfg.pop("extra_kwargs", {})
    c = DatasetConfig(dataset_type=name, dataset_format="jsonl", dataset_path=str(path), shuffle=False, packing=False,
                      processor_config={"processor_name": "byte", "processor_type": processor_type}, fps=2, extra_kwargs=extra, **cfg)
    return DATASET_MAPPING[name](c).build()


def test_qwen3_vl_dataset_stamps_videos_with_the_times_of_the_sampled_frames(tmp_path):
    """The Qwen3-VL datasets decode a video together with its metadata; the ``<t seconds>`` stamps in front of
    every temporal step are the mean times of the frames that were actually sampled (8 fps source, 2 fps sampling)."""
    from lmms_engine_b200.datasets.families import Qwen3VLDataset, Qwen3VLIterableDataset

    _write_video(tmp_path / "v.mp4", n_frames=24, fps=8.0)
    rec = {"messages": [{"role": "user", "content": [{"type": "video_url", "video_url": {"url": str(tmp_path / "v.mp4")}},
                                                     {"type": "text", "text": "what happens?"}]},
                        {"role": "assistant", "content": [{"type": "text", "text": "colours change"}]}]}
    ds = _family_dataset(tmp_path, "qwen3_vl", "qwen3_vl", [rec])
    assert isinstance(ds, Qwen3VLDataset)
    frames, meta = ds.load_video_with_metadata(str(tmp_path / "v.mp4"))
    assert meta["fps"] == 8.0 and meta["total_num_frames"] == 24 and len(meta["frame_times"]) == frames.shape[0] == 6
    out = ds[0][0]
    text = ds.processor.tokenizer.decode([t for t in out["input_ids"].tolist() if t < 256])
    times = meta["frame_times"]
    want = [f"<{(times[2 * i] + times[2 * i + 1]) / 2:.1f} seconds>" for i in range(3)]
    assert all(w in text for w in want), (want, text)
    assert out["video_grid_thw"].tolist()[0][0] == 3 and out["position_ids"].shape == (3, out["input_ids"].numel())
    it = _family_dataset(tmp_path, "qwen3_vl_iterable", "qwen3_vl", [rec])
    assert isinstance(it, Qwen3VLIterableDataset)
    assert torch.equal(next(iter(it))[0]["input_ids"], out["input_ids"])


def test_qwen_omni_dataset_chunks_audio_and_interleaves_sound_tracks(tmp_path):
    """A 70 s clip with a 30 s limit becomes three audio placeholders; with ``use_audio_in_video`` the sound track
    found next to a video is interleaved with the video tokens in 2-second chunks and the positions follow the
    audio-visual index."""
    from lmms_engine_b200.models.mrope import omni_positions_one

    _write_wav(tmp_path / "long.wav", 70)
    _write_video(tmp_path / "clip.mp4", n_frames=48, fps=8.0)
    _write_wav(tmp_path / "clip.wav", 6)
    rec_audio = {"messages": [{"role": "user", "content": [{"type": "audio_url", "audio_url": {"url": str(tmp_path / "long.wav")}},
                                                           {"type": "text", "text": "transcribe"}]},
                              {"role": "assistant", "content": [{"type": "text", "text": "a tone"}]}]}
    rec_av = {"messages": [{"role": "user", "content": [{"type": "video_url", "video_url": {"url": str(tmp_path / "clip.mp4")}},
                                                        {"type": "text", "text": "describe"}]},
                           {"role": "assistant", "content": [{"type": "text", "text": "a tone over colours"}]}]}
    ds = _family_dataset(tmp_path, "qwen_omni", "qwen2_5_omni", [rec_audio, rec_av], extra_kwargs={"use_audio_in_video": True})
    a = ds[0][0]
    assert a["audio_values"].shape[0] == 3  # 30 + 30 + 10 seconds
    proc = ds.processor
    ids = a["input_ids"]
    runs = int(((ids == proc.audio_token_id) & (torch.roll(ids, 1) != proc.audio_token_id)).sum())
    assert runs == 3
    b = ds[1][0]
    ids = b["input_ids"]
    lo = int((ids == proc.vision_start).nonzero()[0])
    hi = int((ids == proc.vision_end).nonzero()[0])
    assert ids[lo + 1] == proc.tokenizer.convert_tokens_to_ids("<|audio_bos|>") and ids[hi - 1] == proc.tokenizer.convert_tokens_to_ids("<|audio_eos|>")
    block = ids[lo + 2:hi - 1]
    is_v = block == proc.video_token_id
    assert is_v.any() and (~is_v).any() and set(block.tolist()) == {proc.video_token_id, proc.audio_token_id}
    switches = int((is_v[1:] != is_v[:-1]).sum())
    assert switches >= 3  # several 2-second chunks of each kind alternate
    t, h, w = b["video_grid_thw"].tolist()[0]
    assert int(is_v.sum()) == t * (h // 2) * (w // 2) and b["audio_values"].shape[0] == 1
    want = omni_positions_one(ids.numpy(), proc.image_token_id, proc.video_token_id, proc.audio_token_id, [], b["video_grid_thw"].tolist(),
                              b["second_per_grid_ts"].tolist(), 2, 25.0, 2.0)
    assert np.array_equal(b["position_ids"].numpy(), want)
    # video and audio tokens of one moment share temporal positions
    pos = b["position_ids"][0, lo + 2:hi - 1]
    assert pos[is_v].min() == pos[~is_v].min()
    # without the option the sound track is ignored
    plain = _family_dataset(tmp_path, "qwen_omni_iterable", "qwen2_5_omni", [rec_av])
    c = next(iter(plain))[0]
    assert "audio_values" not in c and int((c["input_ids"] == proc.audio_token_id).sum()) == 0


def test_llava_video_dataset_time_instruction_frame_directories_and_csv(tmp_path):
    from PIL import Image

    _write_video(tmp_path / "v.mp4", n_frames=40, fps=8.0)
    frames_dir = tmp_path / "frames"
    frames_dir.mkdir()
    for i in range(6):
        Image.fromarray(np.full((32, 32, 3), i * 30, dtype=np.uint8)).save(frames_dir / f"{i:04d}.jpg")
    rec = {"messages": [{"role": "user", "content": [{"type": "video_url", "video_url": {"url": str(tmp_path / "v.mp4")}},
                                                     {"type": "text", "text": "what is shown?"}]},
                        {"role": "assistant", "content": [{"type": "text", "text": "grey frames"}]}]}
    rec_dir = {"messages": [{"role": "user", "content": [{"type": "video_url", "video_url": {"url": str(frames_dir)}},
                                                         {"type": "text", "text": "and here?"}]},
                            {"role": "assistant", "content": [{"type": "text", "text": "six frames"}]}]}
    rec_csv = {"video": str(tmp_path / "v.mp4"), "prompt": "caption this", "answer": "a caption"}
    ds = _family_dataset(tmp_path, "llava_video", "llava_video", [rec, rec_dir, rec_csv],
                         extra_kwargs={"frames_upbound": 4, "force_sample": True, "add_time_instruction": True})
    frames, meta = ds.load_video_with_time(str(tmp_path / "v.mp4"), None)
    assert frames.shape[0] == 4 and meta["num_frames"] == 4 and abs(meta["video_time"] - 5.0) < 1e-6
    assert meta["frame_time"].count("s") == 4
    tok = ds.processor.tokenizer
    text = tok.decode([t for t in ds[0][0]["input_ids"].tolist() if t < 256])
    assert "The video lasts for 5.00 seconds, and 4 frames are uniformly sampled from it." in text and meta["frame_time"] in text
    text_dir = tok.decode([t for t in ds[1][0]["input_ids"].tolist() if t < 256])
    assert "The video lasts for 6.00 seconds" in text_dir
    out_csv = ds[2][0]
    text_csv = tok.decode([t for t in out_csv["input_ids"].tolist() if t < 256])
    assert "caption this" in text_csv and "a caption" in text_csv and (out_csv["labels"] != -100).any()


def test_object_storage_serves_images_audio_and_videos(tmp_path):
    """Media named by bucket + blob path go through a storage client: images from memory, audio and videos through a
    cached local copy; a flaky back end is retried, a missing blob raises (so the record is skipped and logged)."""
    from PIL import Image

    from lmms_engine_b200.utils import object_storage as osto

    bucket = tmp_path / "bucket"
    (bucket / "media").mkdir(parents=True)
    Image.fromarray(np.full((40, 40, 3), 90, dtype=np.uint8)).save(bucket / "media" / "a.png")
    _write_wav(bucket / "media" / "a.wav", 1)
    _write_video(bucket / "media" / "a.mp4", n_frames=16, fps=8.0)

    class Flaky(osto.LocalDirectoryClient):
        calls = 0

        def read(self, blob):
            Flaky.calls += 1
            if Flaky.calls % 2:
                raise ConnectionError("transient")
            return super().read(blob)

    osto.register_storage_backend("flaky_test", Flaky)
    rec = {"messages": [{"role": "user", "content": [{"type": "image_url", "image_url": {"url": "media/a.png"}},
                                                     {"type": "video_url", "video_url": {"url": "media/a.mp4"}},
                                                     {"type": "text", "text": "hi"}]},
                        {"role": "assistant", "content": [{"type": "text", "text": "ok"}]}]}
    ds = _family_dataset(tmp_path, "vision", "qwen2_5_vl", [rec], object_storage="flaky_test", bucket_name=str(bucket),
                         extra_kwargs={"object_cache_dir": str(tmp_path / "cache")})
    import lmms_engine_b200.utils.object_storage as mod

    old = mod.time.sleep
    mod.time.sleep = lambda s: None
    try:
        out = ds[0][0]
        wav, sr = ds.load_audio("media/a.wav")
        with pytest.raises(IOError):
            ds.load_image("media/missing.png")
    finally:
        mod.time.sleep = old
    assert "pixel_values" in out and "pixel_values_videos" in out and len(wav) == sr
    assert len(os.listdir(tmp_path / "cache")) == 2  # the video and the audio clip
    with pytest.raises(ValueError, match="bucket_name"):
        osto.make_client("gcs", None)


def test_dataset_sources_load_in_worker_processes_or_threads(tmp_path):
    from lmms_engine_b200.utils.data_utils import DataUtilities

    specs = []
    for i in range(3):
        path = tmp_path / f"s{i}.jsonl"
        path.write_text("".join(json.dumps({"id": f"{i}-{j}"}) + "\n" for j in range(5)))
        specs.append({"path": str(path), "data_type": "jsonl", "data_folder": f"f{i}"})
    threads = DataUtilities.load_inline_datasets(specs, processes=False)
    procs = DataUtilities.load_inline_datasets(specs, processes=True)
    assert threads == procs and [r["id"] for r in procs[0]][::5] == ["0-0", "1-0", "2-0"] and procs[1][::5] == ["f0", "f1", "f2"]
