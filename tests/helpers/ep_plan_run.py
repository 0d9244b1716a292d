"""Expert-parallel PLANS on CPU/gloo ranks: for every mixture-of-experts family the registered plan
shards the experts over the ep mesh, wraps the rest (towers included) with FSDP2, and the sharded
model reproduces the loss of the unsharded model on this rank's batch."""
import os
import sys
import types

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import torch
import torch.distributed as dist

TEXT = dict(vocab_size=300, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
            num_key_value_heads=2, head_dim=16, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32,
            decoder_sparse_step=1, norm_topk_prob=True, mlp_only_layers=[], router_aux_loss_coef=0.0,
            tie_word_embeddings=False)
VIS = dict(depth=2, hidden_size=32, intermediate_size=64, num_heads=2, patch_size=4, temporal_patch_size=2, spatial_merge_size=2,
           out_hidden_size=64, num_position_embeddings=16, deepstack_visual_indexes=[0], in_channels=3)
LINEAR = dict(linear_conv_kernel_dim=4, linear_key_head_dim=16, linear_value_head_dim=16, linear_num_key_heads=2,
              linear_num_value_heads=4, partial_rotary_factor=0.5, num_hidden_layers=4)


def family_configs():
    mrope = {"rope_scaling": {"mrope_section": [4, 2, 2], "mrope_interleaved": True}}
    yield "qwen3_moe", dict(TEXT)
    yield "qwen3_5_moe_text", dict(TEXT, **LINEAR)
    yield "qwen3_vl_moe", dict(model_type="qwen3_vl_moe", text_config=dict(TEXT, **mrope), vision_config=VIS, image_token_id=290,
                               video_token_id=291, vision_start_token_id=293)
    aud = dict(num_mel_bins=16, d_model=32, encoder_layers=1, encoder_attention_heads=4, encoder_ffn_dim=64, max_source_positions=100,
               n_window=50, n_window_infer=200, output_dim=64, downsample_hidden_size=8, conv_chunksize=3)
    yield "qwen3_omni_moe_thinker", dict(text_config=dict(TEXT, **mrope), vision_config=VIS, audio_config=aud, image_token_id=290,
                                         video_token_id=291, audio_token_id=292, audio_start_token_id=294, vision_start_token_id=293,
                                         position_id_per_seconds=13)
    audio = dict(hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=2, head_dim=16, num_mel_bins=8,
                 sliding_window=6)
    yield "aero_realtime", dict(model_type="aero_realtime", backbone_family="qwen3_vl_moe", text_config=dict(TEXT, **mrope),
                                vision_config=VIS, audio_config=audio, downsample_factor=2, image_token_index=290,
                                video_token_index=291, audio_token_index=292, vision_start_token_index=293)


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    from torch.distributed.tensor import DTensor

    from lmms_engine_b200.mapping_func import create_model_from_config
    from lmms_engine_b200.models.moe_lm import SparseMoeBlock
    from lmms_engine_b200.parallel.parallelize import apply_parallelize, has_parallel_plan
    from lmms_engine_b200.parallel.process_group_manager import setup_process_group_manager

    ep = int(sys.argv[1]) if len(sys.argv) > 1 else world  # ep < world: the experts are also FSDP-sharded over the other ranks
    setup_process_group_manager(tp_size=1, cp_size=1, pp_size=1, dp_size=world, ep_size=ep, device_type="cpu")
    args = types.SimpleNamespace(fsdp_config={"reshard_after_forward": True}, reduce_dtype="float32", output_dtype="float32")
    done = []
    for family, cfg in family_configs():
        if ep < world and family not in ("qwen3_moe", "qwen3_vl_moe"):
            continue
        assert has_parallel_plan(family), family
        torch.manual_seed(0)
        full = create_model_from_config(family, dict(cfg)).float().train()
        torch.manual_seed(0)
        model = create_model_from_config(family, dict(cfg)).float().train()
        apply_parallelize(model, family, args, torch.float32)
        blocks = [m for m in model.modules() if isinstance(m, SparseMoeBlock)]
        assert blocks and all(b.ep is not None for b in blocks), family
        for b in blocks:
            p = b.experts.gate_up_proj
            assert isinstance(p, DTensor) and p.to_local().shape[0] == TEXT["num_experts"] // ep, (family, type(p))
        g = torch.Generator().manual_seed(11 + rank)
        n = 60 + 9 * rank
        ids = torch.randint(0, 280, (1, n), generator=g)
        batch = dict(input_ids=ids, attention_mask=torch.ones_like(ids), labels=ids)
        if family in ("qwen3_moe", "qwen3_5_moe_text"):
            batch = dict(input_ids=ids[0], labels=ids[0], cu_seqlens=torch.tensor([0, 25, n], dtype=torch.int32))
        loss = model(**batch)["loss"]
        loss.backward()
        ref = full(**batch)["loss"]
        assert abs(float(loss) - float(ref)) < 2e-4, (family, float(loss), float(ref))
        grads = [p.grad for p in model.parameters() if p.grad is not None]
        assert len(grads) > 10, family
        # the gradient of the MEAN of the ranks' losses, for expert and non-expert parameters alike
        ref.backward()
        want = {}
        for name, q in full.named_parameters():
            gq = (q.grad if q.grad is not None else torch.zeros_like(q)).clone()
            dist.all_reduce(gq)
            want[name] = gq / world
        checked = 0
        for name, p in model.named_parameters():
            if "experts." not in name or p.grad is None:
                continue
            got = p.grad.full_tensor() if hasattr(p.grad, "full_tensor") else p.grad
            assert got.shape == want[name].shape, (family, name, got.shape, want[name].shape)
            err = float((got - want[name]).abs().max())
            assert err < 2e-4 * max(1.0, float(want[name].abs().max())), (family, name, err)
            checked += 1
        assert checked >= 2, family
        done.append(family)
    # bf16 policy: FSDP must hand the step's context to every wrapped block untouched (fp32 rotary tables, ONE aux list)
    torch.manual_seed(0)
    cfg = dict(TEXT, router_aux_loss_coef=0.01)
    model = create_model_from_config("qwen3_moe", cfg).train()
    apply_parallelize(model, "qwen3_moe", args, torch.bfloat16)
    seen = []
    for layer in model.model.layers:
        layer.self_attn.register_forward_pre_hook(lambda m, a: seen.append((a[1].cos.dtype, id(a[1].aux))))
    ids = torch.randint(0, 280, (70,), generator=torch.Generator().manual_seed(3 + rank))
    out = model(input_ids=ids, labels=ids, cu_seqlens=torch.tensor([0, 30, 70], dtype=torch.int32))
    assert len(seen) == 2 and all(d == torch.float32 for d, _ in seen), seen
    assert len({i for _, i in seen}) == 1 and len(out["aux"]) == 2, (seen, len(out["aux"]))
    out["loss"].backward()
    if rank == 0:
        print("expert parallel plans ok: " + " ".join(done))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
