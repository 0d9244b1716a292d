"""Small host-side components: LPT planner, eval backend with a fake client, CUDA-event
profiler with fake events, schedulers, FLOPs counter, override grammar, merger consolidation."""
import json
import os
import sys
import time

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def test_lpt_planner_balances_and_prefers_home():
    from lmms_engine_b200.parallel.vit_parallel import lpt_balance, plan_frame_exchange

    owner, load = lpt_balance([100, 100, 100, 100], [0, 0, 0, 0], 2)
    assert sorted(load) == [200, 200]
    owner2, _ = lpt_balance([10, 10, 10, 10], [0, 1, 2, 3], 4)
    assert owner2 == [0, 1, 2, 3]  # already balanced: nothing moves
    frames = [[1024] * 6, [1024], [], [256, 256]]
    own, send, load = plan_frame_exchange(frames)
    assert sum(load) == sum(sum(f) for f in frames) and max(load) - min(load) <= 1024
    assert plan_frame_exchange(frames) == (own, send, load)  # deterministic


def test_eval_backend_with_fake_server():
    from lmms_engine_b200.eval.backends import EvalServerBackend

    class FakeClient:
        def __init__(self):
            self.n = 0
            self.payloads = []

        def submit(self, payload):
            self.payloads.append(payload)
            self.n += 1
            return f"job{self.n}"

        def status(self, job):
            if job == "job1":
                return {"status": "completed", "result": {"results": {"mmmu_val": {"acc,none": 0.41, "acc_stderr,none": 0.01}}}}
            return {"status": "failed", "error": "boom"}

    fake = FakeClient()
    be = EvalServerBackend({"server_url": "http://x", "poll_interval": 0.05, "tasks": ["mmmu_val"], "checkpoint_key": "pretrained",
                            "model_args": {"tensor_parallel_size": 1}}, client=fake)
    be.submit("/ckpt/checkpoint-10", 10)
    be.submit("/ckpt/checkpoint-20", 20)
    assert fake.payloads[0]["model_args"]["pretrained"] == "/ckpt/checkpoint-10"
    deadline = time.time() + 5
    results = []
    while time.time() < deadline and be.pending():
        time.sleep(0.05)
    results = list(be.poll_results())
    be.close()
    assert results == [(10, {"eval/mmmu_val_acc": 0.41})]  # the failed job is dropped, not raised


def test_cuda_event_profiler_with_fake_events(tmp_path, monkeypatch):
    from lmms_engine_b200.utils import profiler as prof

    class FakeEvent:
        clock = 0.0

        def __init__(self, enable_timing=True):
            self.t = None

        def record(self):
            FakeEvent.clock += 1.5
            self.t = FakeEvent.clock

        def query(self):
            return True

        def synchronize(self):
            pass

        def elapsed_time(self, other):
            return other.t - self.t

    monkeypatch.setattr(torch.cuda, "is_available", lambda: True)
    monkeypatch.setattr(torch.cuda, "Event", FakeEvent)
    p = prof.CudaEventProfiler(True, str(tmp_path), {"start_step": 1, "end_step": 6, "stride": 2, "ranks": [0]}, rank=0)
    for step in range(8):
        p.set_step(step)
        p.start("training_step")
        p.stop("training_step")
        p.flush()
    p.close()
    lines = [json.loads(l) for l in open(tmp_path / "cuda_event_profiler" / "cuda_events_rank_0.jsonl")]
    assert [l["step"] for l in lines] == [1, 3, 5] and all(l["ms"] == 1.5 for l in lines)
    off = prof.CudaEventProfiler(True, str(tmp_path), {"ranks": [1]}, rank=0)
    assert not off.enable


def test_schedules():
    from lmms_engine_b200.utils.schedulers import lr_factor

    assert lr_factor("cosine", 0, 10, 100) == 0.0 and lr_factor("cosine", 10, 10, 100) == 1.0
    assert abs(lr_factor("cosine", 100, 10, 100, min_lr_ratio=0.1) - 0.1) < 1e-9
    assert lr_factor("wsd", 50, 10, 100, stable_ratio=0.9) == 1.0
    assert lr_factor("wsd", 100, 10, 100, stable_ratio=0.9, min_lr_ratio=0.2) == pytest.approx(0.2)
    assert lr_factor("constant", 0, 10, 100) == pytest.approx(0.01) and lr_factor("constant", 10, 10, 100) == 1.0


def test_flops_formula_matches_reference_definition():
    from lmms_engine_b200.models.utils import FlopsCounter

    cfg = dict(hidden_size=3584, intermediate_size=18944, num_hidden_layers=28, num_attention_heads=28, num_key_value_heads=4,
               head_dim=128, vocab_size=152064)
    fc = FlopsCounter(cfg)
    dense = 28 * (3584 * 18944 * 3 + 3584 * (3584 + 512 + 512 + 3584)) + 2 * 152064 * 3584
    assert fc.dense_params() == dense
    seq = [4096, 8192, 4096]
    assert fc.flops_per_step(seq) == 6.0 * dense * 16384 + 12.0 * sum(s * s for s in seq) * 128 * 28 * 28


def test_override_grammar(tmp_path):
    from lmms_engine_b200.launch import cli

    y = tmp_path / "c.yaml"
    y.write_text("trainer_type: hf_trainer\ntrainer_args:\n  output_dir: /tmp/x\n  max_steps: 5\n")
    cfg = cli.build_config([f"config_yaml={y}", "hydra.output_subdir=null", "hydra/job_logging=disabled"])
    assert cfg["trainer_type"] == "hf_trainer" and cfg["trainer_args"] == {"output_dir": "/tmp/x", "max_steps": 5}
    cfg = cli.build_config(["trainer_args.learning_rate=3e-4", "+trainer_args.custom=[1,2]", "~trainer_args.run_name",
                            "dataset_config.packing=true"])
    assert cfg["trainer_args"]["learning_rate"] == pytest.approx(3e-4) and cfg["trainer_args"]["custom"] == [1, 2]
    assert "run_name" not in cfg["trainer_args"] and cfg["dataset_config"]["packing"] is True
    d = tmp_path / "conf"
    d.mkdir()
    (d / "mine.yaml").write_text("trainer_type: sit_trainer\n")
    assert cli.build_config(["--config-path", str(d), "--config-name", "mine"])["trainer_type"] == "sit_trainer"


def test_consolidate_multi_axis_and_uneven():
    from lmms_engine_b200.merger.consolidate import fold_axis

    full = torch.arange(7 * 4.0).view(7, 4)
    # uneven Shard(0) over 4 ranks: chunks of 2,2,2,1
    pieces = list(torch.chunk(full, 4, 0))
    assert torch.equal(fold_axis(pieces, ("S", 0)), full)
    # 2-D mesh (2 x 2): outer Shard(0), inner Shard(1)
    outer = torch.chunk(full, 2, 0)
    grid = [list(torch.chunk(o, 2, 1)) for o in outer]
    rows = [fold_axis(g, ("S", 1)) for g in grid]
    assert torch.equal(fold_axis(rows, ("S", 0)), full)
    # replicate axis takes one copy; zero-size shard on an axis is skipped
    assert torch.equal(fold_axis([full, full], ("R",)), full)
    assert torch.equal(fold_axis([full, full.new_empty((0, 4))], ("S", 0)), full)


def test_example_configs_parse_into_config_objects():
    """Every shipped example YAML must be accepted by the CLI config builder and the config classes."""
    import glob

    from lmms_engine_b200.datasets.config import DatasetConfig
    from lmms_engine_b200.launch import cli
    from lmms_engine_b200.models.config import ModelConfig
    from lmms_engine_b200.train.config import TrainingArguments
    from lmms_engine_b200.train.registry import TRAINER_REGISTER
    import lmms_engine_b200.train  # noqa: F401  (registers the trainers)

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    files = sorted(glob.glob(os.path.join(root, "examples", "*", "*.yaml")) + glob.glob(os.path.join(root, "examples", "*.yaml")))
    files = [f for f in files if os.sep + "data" + os.sep not in f]
    assert len(files) >= 5
    known = set(TrainingArguments.field_names())
    for f in files:
        cfg = cli.build_config([f"config_yaml={f}"])
        DatasetConfig(**cfg["dataset_config"])
        ModelConfig(**cfg["model_config"])
        assert cfg["trainer_type"] in TRAINER_REGISTER, (f, cfg["trainer_type"])
        unknown = set(cfg["trainer_args"]) - known
        assert not unknown, (f, unknown)
        TrainingArguments(**cfg["trainer_args"])
        # every component an example names is registered, and in-line model configurations parse
        from lmms_engine_b200 import mapping_func as mf
        import lmms_engine_b200.datasets.registry  # noqa: F401

        assert cfg["dataset_config"]["dataset_type"] in mf.DATASET_MAPPING, f
        assert cfg["dataset_config"]["processor_config"]["processor_type"] in mf.DATAPROCESSOR_MAPPING, f
        inline = cfg["model_config"].get("load_from_config")
        if inline:
            config_cls = mf._resolve(inline["model_type"], None)[0]
            parsed = config_cls.from_dict(dict(inline["config"], model_type=inline["model_type"]))
            stray = set(getattr(parsed, "extra", None) or {}) - {"model_type"}
            assert not stray, (f, stray)


def test_tools_and_legacy_merge(tmp_path):
    from lmms_engine_b200.merger import legacy
    from lmms_engine_b200.tools import check_data, create_json_dataset, generate_default_yaml

    out = tmp_path / "d.yaml"
    generate_default_yaml.main(["--output", str(out)])
    import yaml

    cfg = yaml.safe_load(open(out))
    assert cfg["trainer_type"] == "fsdp2_trainer" and "learning_rate" in cfg["trainer_args"]
    # qa records -> messages -> check
    src = tmp_path / "qa.jsonl"
    src.write_text(json.dumps({"question": "what is this", "answer": "a cat", "image": "cat.png"}) + "\n")
    create_json_dataset.main(["--input", str(src), "--output", str(tmp_path / "m.jsonl")])
    rows = [json.loads(l) for l in open(tmp_path / "m.jsonl")]
    rep = check_data.check(rows, str(tmp_path))
    assert rep["rows"] == 1 and rep["media"] == {"image_url": 1} and rep["missing"] == [(0, "cat.png")]
    assert rep["tokens_total"] >= 2000
    # two "checkpoints" of dim-0 sharded tensors -> merged and averaged
    for step, val in ((10, 1.0), (20, 3.0)):
        d = tmp_path / "run" / f"checkpoint-{step}" / "pytorch_model_fsdp_0"
        d.mkdir(parents=True)
        for r in range(2):
            torch.save({"w": torch.full((2, 3), val + r), "b": torch.full((1,), val)}, d / f"model_world_size_2_rank_{r}.pt")
    one = legacy.merge_fsdp2_dir(str(tmp_path / "run" / "checkpoint-10"))
    assert one["w"].shape == (4, 3) and one["w"][3, 0] == 2.0
    out_dir = legacy.main(["--input_dir", str(tmp_path / "run"), "--merge", "--dtype", "float32"])
    from lmms_engine_b200.models import hf_io

    merged = hf_io.read_state_dict(str(out_dir))
    assert torch.allclose(merged["w"][:2], torch.full((2, 3), 2.0)) and torch.allclose(merged["w"][2:], torch.full((2, 3), 3.0))


def test_monkey_patcher_registry_runs_user_patches():
    from lmms_engine_b200.models.monkey_patch import MONKEY_PATCHER

    seen = []

    @MONKEY_PATCHER.register("my_model", "liger")
    def patch(model, rms_norm=True, **kw):
        seen.append((model, rms_norm))

    assert MONKEY_PATCHER.apply("m", "my_model", ["liger", "other"], rms_norm=False) == 1
    assert seen == [("m", False)] and MONKEY_PATCHER.apply("m", "unknown", "liger") == 0


def test_head_routing_tables_match_the_ulysses_layout():
    """Routing tables of the fused QKV projection against the reference layout: scattering the columns of
    ``[q | k | v]`` by the tables must equal what the NCCL all-to-all path builds."""
    from lmms_engine_b200.parallel.fused_comm import out_head_route, qkv_head_route, qkv_kb_sources

    nq, nkv, D, world = 8, 4, 128, 4
    r = qkv_head_route(nq, nkv, D, world, "cpu")
    hq, hkv = nq // world, nkv // world
    assert r.cols_local == (hq + 2 * hkv) * D and not r.kv_replicated
    n_chunks = (nq + 2 * nkv) * D // 64
    assert r.chunk_dst.numel() == n_chunks
    # emulate the scatter on column ids: value = global column index
    cols = torch.arange((nq + 2 * nkv) * D)
    got = {d: torch.full((r.cols_local,), -1, dtype=torch.long) for d in range(world)}
    for c in range(n_chunks):
        for dd in range(int(r.chunk_ndst[c])):
            d = int(r.chunk_dst[c]) + dd
            got[d][int(r.chunk_col[c]):int(r.chunk_col[c]) + 64] = cols[c * 64:(c + 1) * 64]
    for d in range(world):
        q = cols[: nq * D].view(nq, D)[d * hq:(d + 1) * hq].reshape(-1)
        k = cols[nq * D:(nq + nkv) * D].view(nkv, D)[d * hkv:(d + 1) * hkv].reshape(-1)
        v = cols[(nq + nkv) * D:].view(nkv, D)[d * hkv:(d + 1) * hkv].reshape(-1)
        assert torch.equal(got[d], torch.cat([q, k, v]))
    # k-block sources follow the owner of every head
    kb = qkv_kb_sources(nq, nkv, D, world, "cpu")
    assert kb.tolist()[: nq * D // 64] == [h // hq for h in range(nq) for _ in range(D // 64)]
    # replicated kv heads: each kv head goes to world / n_kv consecutive ranks
    rr = qkv_head_route(8, 2, 64, 4, "cpu")
    assert rr.kv_replicated and rr.chunk_ndst.tolist() == [1] * 8 + [2] * 4 and rr.chunk_dst.tolist()[8:] == [0, 2, 0, 2]
    o = out_head_route(nq, D, world, "cpu")
    assert o.cols_local == hq * D and o.chunk_dst.tolist() == [h // hq for h in range(nq) for _ in range(2)]
    with pytest.raises(ValueError):
        qkv_head_route(28, 4, 128, 8, "cpu")


def test_ema_filter_compute_tracker_and_formatting(tmp_path, monkeypatch):
    from lmms_engine_b200.utils.compute_tracker import ComputeTracker
    from lmms_engine_b200.utils.ema_utils import EMAHelper
    from lmms_engine_b200.utils.train_utils import TrainUtilities

    model = torch.nn.Sequential(torch.nn.Linear(4, 4), torch.nn.LayerNorm(4))
    model[1].bias.requires_grad_(False)
    ema = EMAHelper(model, decay=0.5, param_filter={"mode": "regex", "include": [r"^0[.]"], "exclude": ["bias"]})
    ema.maybe_init()
    assert sorted(ema.state_dict()) == ["0.weight"]
    w0 = model[0].weight.detach().clone()
    with torch.no_grad():
        model[0].weight.add_(2.0)
    ema.update(1)
    assert torch.allclose(ema.state_dict()["0.weight"].float(), w0 + 1.0, atol=1e-6)  # 0.5 * old + 0.5 * new
    monkeypatch.setattr(TrainUtilities, "_device_name", staticmethod(lambda: "NVIDIA B200"))
    assert TrainUtilities.get_device_flops("P") == pytest.approx(2.25) and TrainUtilities.get_device_tdp() == 1000.0
    ct = ComputeTracker(num_gpus=8)
    ct.update(flops=1e18, tokens=2_000_000, seconds=3600.0)
    s = ct.summary()
    assert s["energy_kwh"] == pytest.approx(8.0) and s["gpu_hours"] == pytest.approx(8.0) and s["total_tokens_human"] == "2.00M"
    assert s["total_flops_human"] == "1.00 EFLOPs" and s["co2_kg"] == pytest.approx(8.0 * 0.475)
    ct2 = ComputeTracker(num_gpus=8)
    ct2.load_state_dict(ct.state_dict())
    assert ct2.summary()["total_flops"] == 1e18
    hf = TrainUtilities.convert_open_to_hf([{"role": "user", "content": [{"type": "image_url", "image_url": {"url": "a.png"}},
                                                                           {"type": "text", "text": "hi"}]}])
    assert hf[0]["content"][0] == {"type": "image", "image": "a.png"}


def test_prepare_init_weight_composes_parts_and_grows_vocabulary(tmp_path):
    """A decoder checkpoint + an audio-encoder checkpoint -> an ``aero`` checkpoint with three more tokens."""
    import torch

    from lmms_engine_b200.mapping_func import create_model_from_config, create_model_from_pretrained
    from lmms_engine_b200.models import hf_io
    from lmms_engine_b200.tools import create_hf_dataset, prepare_init_weight, split_jsonl

    torch.manual_seed(0)
    text = dict(vocab_size=125, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
                num_key_value_heads=2, tie_word_embeddings=False)
    audio = dict(d_model=32, encoder_layers=2, encoder_attention_heads=4, encoder_ffn_dim=64, num_mel_bins=16, max_source_positions=50)
    lm = create_model_from_config("qwen2", dict(text, model_type="qwen2"))
    hf_io.save_pretrained(lm, str(tmp_path / "lm"))
    donor = create_model_from_config("qwen2_audio", dict(model_type="qwen2_audio", text_config=text, audio_config=audio))
    hf_io.save_pretrained({"audio_tower." + k: v for k, v in donor.audio_tower.state_dict().items()}, str(tmp_path / "enc"), config={})
    cfg_path = tmp_path / "aero.json"
    cfg_path.write_text(json.dumps(dict(model_type="aero", text_config=text, audio_config=audio, audio_token_index=126)))
    report = prepare_init_weight.main(["--model-type", "aero", "--config", str(cfg_path), "--part", f"language_model={tmp_path / 'lm'}",
                                       "--part", f"audio_tower={tmp_path / 'enc'}", "--add-tokens", "3", "--pad-vocab-to", "64",
                                       "--dtype", "float32", "--output", str(tmp_path / "out")])
    assert report["language_model"]["placed"] == len(lm.state_dict()) and report["audio_tower"]["unused"] == 0
    assert report["fresh"] >= 1  # the projector
    model = create_model_from_pretrained(str(tmp_path / "out"))
    emb = model.language_model.model.embed_tokens.weight
    assert emb.shape[0] == 128
    assert torch.equal(emb[:125], lm.model.embed_tokens.weight)
    # new rows sit near the mean embedding
    mu = lm.model.embed_tokens.weight.mean(0)
    assert (emb[125:] - mu).abs().max() < 0.05
    assert torch.equal(model.audio_tower.state_dict()["layers.0.self_attn.q_proj.weight"],
                       donor.audio_tower.state_dict()["layers.0.self_attn.q_proj.weight"])
    # the same composition as a family recipe: configs read from the parts' directories, ids continue the vocabulary
    hf_io.save_pretrained({"audio_tower." + k: v for k, v in donor.audio_tower.state_dict().items()}, str(tmp_path / "enc2"),
                          config={"audio_config": audio})
    report = prepare_init_weight.main(["--recipe", "aero", "--language-model", str(tmp_path / "lm"), "--audio-model", str(tmp_path / "enc2"),
                                       "--dtype", "float32", "--output", str(tmp_path / "out_recipe")])
    assert report["language_model"]["placed"] == len(lm.state_dict()) and report["audio_tower"]["unused"] == 0
    again = create_model_from_pretrained(str(tmp_path / "out_recipe"))
    assert again.language_model.model.embed_tokens.weight.shape[0] == 128 and again.config.audio_token_index == 127
    # an autoencoder from a SigLIP checkpoint, configuration only
    enc_cfg = dict(hidden_size=32, intermediate_size=64, num_hidden_layers=1, num_attention_heads=4, image_size=32, patch_size=8)
    (tmp_path / "siglip").mkdir()
    (tmp_path / "siglip" / "config.json").write_text(json.dumps({"vision_config": enc_cfg}))
    prepare_init_weight.main(["--recipe", "rae_siglip2", "--vision-model", str(tmp_path / "siglip"), "--skip-weights", "--noise-tau", "0.5",
                              "--output", str(tmp_path / "rae")])
    rae = json.load(open(tmp_path / "rae" / "config.json"))
    assert rae["model_type"] == "rae_siglip" and rae["encoder_config"]["hidden_size"] == 32 and rae["decoder_config"]["decoder_hidden_size"] == 1152
    # conversation conversion and splitting
    src = tmp_path / "llava.json"
    src.write_text(json.dumps([{"id": "a", "image": "x.png", "conversations": [
        {"from": "human", "value": "<image>\nwhat is it"}, {"from": "gpt", "value": "a cat"}]}] * 5))
    assert create_hf_dataset.main(["--input", str(src), "--output", str(tmp_path / "ds")]) == 5
    rows = [json.loads(l) for l in open(tmp_path / "ds" / "train.jsonl")]
    assert rows[0]["messages"][0]["content"][0]["type"] == "image_url" and rows[0]["messages"][1]["role"] == "assistant"
    parts = split_jsonl.main(["-i", str(tmp_path / "ds" / "train.jsonl"), "-s", "2"])
    assert [sum(1 for _ in open(p)) for p in parts] == [3, 2]


def test_deepspeed_configs_are_rejected_with_directions():
    """A ``deepspeed:`` entry is not silently dropped: the error names the runtimes that replace ZeRO."""
    import pytest

    from lmms_engine_b200.launch.cli import create_train_task

    cfg = {"trainer_type": "fsdp2_trainer", "dataset_config": {"dataset_type": "synthetic_packed", "dataset_format": "synthetic"},
           "model_config": {"load_from_config": {"model_type": "qwen2", "config": {}}},
           "trainer_args": {"output_dir": "/tmp/x", "deepspeed": "examples/ds_config/zero2.json"}}
    with pytest.raises(ValueError, match="native_sharded"):
        create_train_task(cfg)


def test_rank_layout_from_degrees_reports_bad_combinations():
    import pytest

    from lmms_engine_b200.parallel.process_group_manager import RankLayout

    lay = RankLayout.from_degrees(8, tp=2, cp=2)
    assert (lay.dp, lay.tp, lay.cp) == (2, 2, 2)
    with pytest.raises(ValueError, match="cannot be split"):
        RankLayout.from_degrees(8, tp=3)
    with pytest.raises(ValueError, match="positive"):
        RankLayout.from_degrees(8, tp=-1)


def test_length_grouped_sampler_groups_and_shards():
    """Every sample once per epoch, the ranks of a step hold similar lengths, text-only and multimodal samples
    are batched apart, epochs differ, ranks of one data-parallel index agree."""
    import random

    from lmms_engine_b200.train.samplers import LengthGroupedSampler

    rnd = random.Random(0)
    lengths = [rnd.randint(10, 2000) * (1 if rnd.random() < 0.7 else -1) for _ in range(960)]
    R, B = 4, 2
    per_rank = [list(LengthGroupedSampler(lengths, B, num_replicas=R, rank=r, seed=5)) for r in range(R)]
    assert sorted(i for pr in per_rank for i in pr) == list(range(960))
    spreads, mixed = [], 0
    for step in range(len(per_rank[0]) // B):
        idx = [i for pr in per_rank for i in pr[step * B:(step + 1) * B]]
        ls = [abs(lengths[i]) for i in idx]
        spreads.append(max(ls) - min(ls))
        mixed += len({lengths[i] >= 0 for i in idx}) > 1
    assert sum(spreads) / len(spreads) < 150, sum(spreads) / len(spreads)  # a random batch of 8 spreads over ~1500
    assert mixed <= 3
    again = LengthGroupedSampler(lengths, B, num_replicas=R, rank=0, seed=5)
    assert list(again) == per_rank[0]
    again.set_epoch(1)
    assert list(again) != per_rank[0]


def test_check_data_subcommands_measure_media_and_write_precomputed_tokens(tmp_path, capsys):
    """exists / tokens / precompute / summary over a YAML of sources, from folders and through an object-storage client."""
    import wave

    import numpy as np
    import yaml
    from PIL import Image

    from lmms_engine_b200.tools import check_data

    media = tmp_path / "media"
    media.mkdir()
    Image.fromarray(np.zeros((280, 560, 3), dtype=np.uint8)).save(media / "a.png")
    with wave.open(str(media / "s.wav"), "wb") as w:
        w.setnchannels(1), w.setsampwidth(2), w.setframerate(16000)
        w.writeframes(np.zeros(16000 * 2, dtype=np.int16).tobytes())
    rows = [{"id": "r0", "messages": [{"role": "user", "content": [{"type": "image_url", "image_url": {"url": "a.png"}},
                                                                   {"type": "audio_url", "audio_url": {"url": "s.wav"}},
                                                                   {"type": "text", "text": "what is it"}]}]},
            {"messages": [{"role": "user", "content": [{"type": "image_url", "image_url": {"url": "gone.png"}}]}]}]
    data = tmp_path / "d.jsonl"
    data.write_text("".join(json.dumps(r) + "\n" for r in rows))
    spec = tmp_path / "d.yaml"
    spec.write_text(yaml.safe_dump({"datasets": [{"path": str(data), "data_folder": str(media), "data_type": "jsonl"}]}))
    assert check_data.main(["exists", "--dataset", str(spec), "--out", str(tmp_path / "missing.txt")]) == 1
    assert (tmp_path / "missing.txt").read_text().strip().endswith("gone.png")
    assert check_data.main(["tokens", "--dataset", str(spec), "--out", str(tmp_path / "tokens.txt")]) == 0
    image_tokens, audio_tokens, default_image = 280 * 560 // (14 * 14 * 4), 50, 500 * 500 // (14 * 14 * 4)
    assert f"({image_tokens + audio_tokens + default_image})" in (tmp_path / "tokens.txt").read_text()
    assert check_data.main(["precompute", "--dataset", str(spec), "--out-dir", str(tmp_path / "out")]) == 0
    got = [json.loads(l) for l in open(tmp_path / "out" / "d.jsonl")]
    parts = got[0]["messages"][0]["content"]
    assert parts[0]["precomputed_tokens"] == image_tokens and parts[1]["precomputed_tokens"] == audio_tokens
    assert parts[2]["precomputed_tokens"] == 3 * 1.25 and got[1]["id"] == "Unknown_ID"
    assert got[1]["messages"][0]["content"][0]["precomputed_tokens"] == default_image  # unreadable: the default, and reported
    assert "unreadable_media" in capsys.readouterr().out
    assert check_data.estimate_tokens(got[0]) == int(image_tokens + audio_tokens + 3.75)
    # the same through a storage client ("local" = a directory standing in for a bucket), and the single-table form
    cloud = tmp_path / "cloud.yaml"
    cloud.write_text(yaml.safe_dump({"datasets": [{"path": str(data), "data_folder": "", "data_type": "jsonl"}]}))
    assert check_data.main(["precompute", "--dataset", str(cloud), "--parquet", str(tmp_path / "all.parquet"),
                            "--object-storage", "local", "--bucket", str(media)]) == 0
    import pyarrow.parquet as pq

    table = pq.read_table(tmp_path / "all.parquet").to_pylist()
    assert json.loads(table[0]["messages"])[0]["content"][0]["precomputed_tokens"] == image_tokens
    assert check_data.main(["summary", "--dataset", str(spec)]) == 1


def test_sharegpt_conversations_become_messages(tmp_path):
    """``<image>`` in a record that carries a video becomes a video item in front of the turn's text; the parquet holds
    the messages as a JSON string that the map-style dataset reads back."""
    from lmms_engine_b200.tools import convert_sharegpt as cs

    entries = [{"id": 7, "video": "clips/a.mp4", "conversations": [{"from": "human", "value": "<image>\nWhat happens?"},
                                                                   {"from": "gpt", "value": "A cat jumps."},
                                                                   {"from": "human", "value": "And then?"}, {"from": "gpt", "value": "It lands."}]},
               {"id": "b", "image": ["x.png", "y.png"], "conversations": [{"from": "human", "value": "Compare <image> and <image> <image>"},
                                                                          {"from": "gpt", "value": "Same."}]},
               {"id": "bad", "conversations": [{"from": "alien", "value": "?"}]}]
    src = tmp_path / "0_30_s_academic" / "x_oe_processed.json"
    src.parent.mkdir()
    src.write_text(json.dumps(entries))
    (tmp_path / "0_30_s_academic" / "x_mc_processed.json").write_text(json.dumps(entries[:1]))
    out = tmp_path / "out" / "v.parquet"
    cs.main(["--input-dir", str(tmp_path), "--glob", "0_30_s*/*_processed.json", "--contains", "_oe_", "--system", "Watch in silence.",
             "--output", str(out)])
    import pyarrow.parquet as pq

    table = pq.read_table(out).to_pydict()
    assert table["id"] == ["7", "b"]
    first, second = (json.loads(m) for m in table["messages"])
    assert first[0] == {"role": "system", "content": [{"type": "text", "text": "Watch in silence."}]}
    assert first[1]["content"] == [{"type": "video_url", "video_url": {"url": "clips/a.mp4"}}, {"type": "text", "text": "What happens?"}]
    assert [m["role"] for m in first] == ["system", "user", "assistant", "user", "assistant"] and first[3]["content"][0]["text"] == "And then?"
    kinds = [c["type"] for c in second[1]["content"]]
    assert kinds == ["image_url", "image_url", "text"] and second[1]["content"][2]["text"] == "Compare\nand"  # third marker: no media left
    jl = tmp_path / "v.jsonl"
    cs.main(["--input", str(src), "--output", str(jl), "--max-per-file", "1"])
    assert len(jl.read_text().splitlines()) == 1


def test_config_files_and_capability_probes(tmp_path, monkeypatch):
    """JSON and YAML configurations load alike (also by a path relative to the project root) and drive the launcher;
    the capability probes answer without importing anything heavy."""
    from lmms_engine_b200.launch import cli
    from lmms_engine_b200.utils import config_loader as cl
    from lmms_engine_b200.utils import import_utils as iu

    cfg = {"trainer_type": "fsdp2_trainer", "dataset_config": {"dataset_type": "vision", "dataset_format": "json"},
           "model_config": {"load_from_pretrained_path": "x"}, "trainer_args": {"output_dir": "out", "learning_rate": 1e-5}}
    for name in ("a.json", "b.yaml", "c.yml"):
        cl.save_config(cfg, str(tmp_path / "conf" / name))
        assert cl.load_config(str(tmp_path / "conf" / name)) == cfg
    with pytest.raises(ValueError):
        cl.load_config(str(tmp_path / "conf" / "a.json").replace("a.json", "a.txt")) if (tmp_path / "conf" / "a.txt").write_text("x") else None
    with pytest.raises(FileNotFoundError):
        cl.load_config("no/such/file.yaml")
    (tmp_path / "pyproject.toml").write_text("")
    (tmp_path / "deep" / "er").mkdir(parents=True)
    monkeypatch.chdir(tmp_path / "deep" / "er")
    assert cl.load_config("conf/b.yaml") == cfg  # found from the project root
    built = cli.build_config([f"config_yaml={tmp_path / 'conf' / 'a.json'}", "trainer_args.learning_rate=2e-5"])
    assert built["trainer_type"] == "fsdp2_trainer" and built["trainer_args"]["output_dir"] == "out"
    assert built["trainer_args"]["learning_rate"] == 2e-5 and "config_yaml" not in built  # the command line has the last word
    assert iu.is_package_available("torch") and not iu.is_package_available("surely_not_a_package")
    assert iu.is_torch_version_greater_than("1.0") and iu.is_transformers_version_greater_or_equal_to("4.0")
    assert iu.is_torch_npu_available() is False and isinstance(iu.is_video_audio_available(), bool)
    if not torch.cuda.is_available():
        assert not iu.is_flash_attn_2_available() and not iu.is_liger_kernel_available() and not iu.is_fused_moe_available()


def test_public_class_names_of_the_reference_resolve():
    """``from lmms_engine.<package> import <Name>`` works for the names the reference exports from its datasets, models,
    train and utils packages; a custom dataset can subclass ``BaseDataset`` and register itself."""
    import importlib

    import torch

    exported = {
        "lmms_engine.datasets": ["DatasetConfig", "MultiModalDataset", "VisionSFTDataset", "VisionAudioSFTDataset", "FinewebEduDataset",
                                 "MultiModalIterableDataset", "VisionSFTIterableDataset"],
        "lmms_engine.datasets.naive": ["BaseDataset", "QwenOmniSFTDataset", "Qwen3VLDataset", "RaeDataset", "SitDataset", "LLaVAVideoDataset"],
        "lmms_engine.datasets.iterable": ["AeroRealtimeIterableDataset", "BaseIterableDataset", "BagelIterableDataset", "LlavaOv2IterableDataset",
                                          "Qwen3VLIterableDataset", "QwenOmniIterableDataset"],
        "lmms_engine.datasets.collator": ["AeroRealtimeCollator", "VisionCollator", "BagelCollator", "LLaVACollator"],
        "lmms_engine.datasets.processor": ["ProcessorConfig", "AeroDataProcessor", "AeroRealtimeDataProcessor", "BaseQwen2_5_DataProcessor",
                                           "LLaVADataProcessor", "LLaVAVideoDataProcessor", "NanovlmDataProcessor", "Qwen2_5OmniDataProcessor",
                                           "Qwen3OmniMoeDataProcessor", "Qwen2_5_VLDataProcessor", "Qwen2VLDataProcessor", "WanVideoDataProcessor",
                                           "PureTextDataProcessor", "Qwen2DataProcessor", "BagelDataProcessor", "RaeSiglipDataProcessor",
                                           "SitDataProcessor", "Qwen3_VLDataProcessor", "LlavaOnevision2DataProcessor"],
        "lmms_engine.models": ["AeroForConditionalGeneration", "AeroConfig", "AeroRealtimeConfig", "AeroRealtimeForConditionalGeneration",
                               "AeroRealtimeProcessor", "Bagel", "BagelConfig", "ModelConfig", "AeroProcessor", "MONKEY_PATCHER",
                               "Qwen2_5OmniThinkerConfig", "Qwen2_5OmniThinkerForConditionalGeneration", "Qwen3OmniMoeThinkerConfig",
                               "Qwen3OmniMoeThinkerForConditionalGeneration", "WanVideoConfig", "WanVideoForConditionalGeneration",
                               "WanVideoProcessor", "NanovlmConfig", "NanovlmForConditionalGeneration", "RaeSiglipConfig", "RaeSiglipModel",
                               "SiTModel", "SiTConfig", "SiT", "Qwen3DLLMForMaskedLM", "DreamDLLMConfig", "LLaDADLLMForMaskedLM",
                               "Llavaonevision1_5Config", "LLaVAOneVision1_5_ForConditionalGeneration", "apply_liger_kernel_to_qwen3",
                               "apply_liger_kernel_to_qwen3_vl_moe", "apply_liger_kernel_to_aero_realtime"],
        "lmms_engine.train": ["TrainerConfig", "Trainer", "TrainingArguments", "TrainRunner", "TRAINER_REGISTER", "FSDP2SFTTrainer", "DLLMTrainer",
                              "WanVideoTrainer"],
        "lmms_engine.utils": ["Logging", "DataUtilities", "TrainUtilities", "StepProfiler", "ComputeTracker"],
        "lmms_engine.protocol": ["Runnable", "Processable", "SFTChatData", "Args"],
        "lmms_engine.merger": ["CheckpointMerger", "FSDP2Merger"],
    }
    for module, names in exported.items():
        mod = importlib.import_module(module)
        for name in names:
            assert getattr(mod, name) is not None, (module, name)
    with pytest.raises(AttributeError):
        importlib.import_module("lmms_engine.datasets.naive").NoSuchDataset

    from lmms_engine.datasets.collator import LLaVACollator
    from lmms_engine.datasets.naive import BaseDataset
    from lmms_engine.mapping_func import DATASET_MAPPING, register_dataset
    from lmms_engine.models import MONKEY_PATCHER, apply_liger_kernel_to_qwen3

    @register_dataset("my_custom_records")
    class Mine(BaseDataset):
        pass

    assert DATASET_MAPPING.pop("my_custom_records") is Mine and hasattr(Mine, "get_collator") and hasattr(Mine, "build")
    seen = []
    MONKEY_PATCHER.register("qwen3", "liger")(lambda model, **kw: seen.append((model, kw)))
    try:
        assert apply_liger_kernel_to_qwen3() == 0 and apply_liger_kernel_to_qwen3(model="m", rope=True) == 1
        assert seen == [("m", {"rope": True})]
    finally:
        MONKEY_PATCHER._patches.pop(("qwen3", "liger"))
    batch = LLaVACollator(pad_token_id=0)([
        {"input_ids": torch.arange(1, 4), "labels": torch.arange(1, 4), "pixel_values": torch.ones(1, 3, 2, 2, 2), "use_audio_in_video": False},
        {"input_ids": torch.arange(1, 6), "labels": torch.arange(1, 6), "pixel_values": torch.ones(1, 5, 2, 2, 2), "use_audio_in_video": False}])
    assert batch["pixel_values"].shape == (2, 5, 2, 2, 2) and batch["pixel_values"][0, 3:].abs().sum() == 0
    assert batch["use_audio_in_video"] is False and batch["attention_mask"].sum(1).tolist() == [3, 5]
