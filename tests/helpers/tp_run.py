"""Tensor-parallel (sequence-parallel flavour) and Ulysses checks on CPU/gloo ranks against
the unsharded model: same loss, same gradients."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import torch
import torch.distributed as dist


def vl_deepstack(mode):
    """Qwen3-VL style model (deepstack features added at visual positions) with the token stream split over a
    Ulysses group or a tensor-parallel group: same loss as the unsharded model."""
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    from torch.distributed.device_mesh import init_device_mesh

    from lmms_engine_b200.mapping_func import create_model_from_config
    from lmms_engine_b200.parallel.tensor_parallel import shard_decoder_for_tp

    text = dict(vocab_size=300, hidden_size=64, intermediate_size=128, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2,
                head_dim=16, tie_word_embeddings=False, rope_scaling={"mrope_section": [4, 2, 2], "mrope_interleaved": True})
    vis = dict(depth=2, hidden_size=32, intermediate_size=64, num_heads=2, patch_size=4, temporal_patch_size=2, spatial_merge_size=2,
               out_hidden_size=64, num_position_embeddings=16, deepstack_visual_indexes=[0, 1], in_channels=3)
    cfg = dict(model_type="qwen3_vl", text_config=text, vision_config=vis, image_token_id=290, video_token_id=291, vision_start_token_id=293)
    torch.manual_seed(0)
    full = create_model_from_config("qwen3_vl", dict(cfg)).float()
    torch.manual_seed(0)
    model = create_model_from_config("qwen3_vl", dict(cfg)).float()
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(0, 280, (1, 61), generator=g)  # odd length: the split pads
    ids[0, 2], ids[0, 3:7] = 293, 290
    ids[0, 30], ids[0, 31:47] = 293, 290
    pix = torch.randn(16 + 64, 3 * 2 * 4 * 4, generator=g)
    grid = torch.tensor([[1, 4, 4], [1, 8, 8]])
    batch = dict(input_ids=ids, attention_mask=torch.ones_like(ids), labels=ids, pixel_values=pix, image_grid_thw=grid)
    ref = full(**batch)["loss"]
    if mode == "vl_ulysses":
        model.sp_group = dist.group.WORLD
    else:
        mesh = init_device_mesh("cpu", (world,), mesh_dim_names=("tp",))
        shard_decoder_for_tp(model.language_model, mesh, mesh.get_group())
    loss = model(**batch)["loss"]
    loss.backward()
    assert abs(float(loss) - float(ref)) < 1e-4, (mode, float(loss), float(ref))
    if mode == "vl_ulysses":
        # every rank ran the tower on its share of the images (two images, two ranks); the mean of the ranks' gradients
        # (what the data-parallel reduction computes) is the full model's gradient, for the tower and for the decoder
        ref.backward()
        for (name, p), (_, q) in zip(model.named_parameters(), full.named_parameters()):
            g = (p.grad if p.grad is not None else torch.zeros_like(p)).clone()
            dist.all_reduce(g)
            g /= world
            want = q.grad if q.grad is not None else torch.zeros_like(q)
            assert (g - want).abs().max() < 2e-4 * max(1.0, float(want.abs().max())), (name, float((g - want).abs().max()))
        model.sp_split_vit = False  # every rank runs the whole tower: same loss
        again = model(**batch)["loss"]
        assert abs(float(again) - float(ref)) < 1e-4
    if rank == 0:
        print(f"{mode} ok")
    dist.destroy_process_group()


def main(mode):
    if mode.startswith("vl_"):
        return vl_deepstack(mode)
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    from torch.distributed.device_mesh import init_device_mesh

    from lmms_engine_b200.models.decoder_lm import DecoderConfig, DecoderLM
    from lmms_engine_b200.parallel import tp_ops
    from lmms_engine_b200.parallel.tensor_parallel import shard_decoder_for_tp

    cfg = DecoderConfig(model_type="qwen3", vocab_size=256, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                        num_attention_heads=4, num_key_value_heads=2 if mode == "tp" else 1, head_dim=16)
    build = DecoderLM
    if mode.startswith("ulysses_hybrid"):
        # Gated-DeltaNet + gated-attention hybrid: both layer kinds trade the sequence split for a head split; in the
        # "_state" variant the linear-attention layers keep their tokens and hand the recurrent state from rank to rank
        # (3 key heads / 3 value heads: no head split over 2 or 4 ranks exists)
        from lmms_engine_b200.models.qwen3_5 import Qwen35Config, Qwen35LM

        state = mode.endswith("_state")
        cfg = Qwen35Config(vocab_size=256, hidden_size=64, intermediate_size=128, num_hidden_layers=4, num_attention_heads=4,
                           num_key_value_heads=2 if not state else 4, head_dim=16, linear_conv_kernel_dim=4, linear_key_head_dim=16,
                           linear_value_head_dim=16, linear_num_key_heads=3 if state else 2, linear_num_value_heads=3 if state else 4,
                           partial_rotary_factor=0.5, linear_attn_cp="state" if state else "auto")
        build = Qwen35LM
    torch.manual_seed(0)
    full = build(cfg)
    torch.manual_seed(0)
    model = build(cfg)
    if mode.startswith("ulysses_hybrid"):
        with torch.no_grad():  # zero-centred norm scales and unit decay parameters would hide mistakes
            for m_ in (full, model):
                g_ = torch.Generator().manual_seed(7)
                for p_ in m_.parameters():
                    if p_.dim() == 1:
                        p_.copy_(0.5 * torch.rand(p_.shape, generator=g_))
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(0, 256, (91,), generator=g)  # not a multiple of the group size: exercises padding
    cu = torch.tensor([0, 40, 91], dtype=torch.int32)
    if mode.endswith("_state"):  # a document that spans three ranks' slices, then two short ones
        ids = torch.randint(0, 256, (203,), generator=g)
        cu = torch.tensor([0, 150, 170, 203], dtype=torch.int32)
    ref = full(input_ids=ids, labels=ids, cu_seqlens=cu)["loss"]
    ref.backward()
    if mode == "tp":
        mesh = init_device_mesh("cpu", (world,), mesh_dim_names=("tp",))
        shard_decoder_for_tp(model, mesh, mesh.get_group())
        loss = model(input_ids=ids, labels=ids, cu_seqlens=cu)["loss"]
        loss.backward()
        tp_ops.sync_replicated_grads(model, mesh.get_group())
        assert abs(float(loss) - float(ref)) < 1e-4, (float(loss), float(ref))
        for (n, p), (_, pf) in zip(model.named_parameters(), full.named_parameters()):
            gr = p.grad.full_tensor() if hasattr(p.grad, "full_tensor") else p.grad
            assert torch.allclose(gr, pf.grad, atol=2e-4), (n, (gr - pf.grad).abs().max())
    else:  # ulysses
        model.sp_group = dist.group.WORLD
        loss = model(input_ids=ids, labels=ids, cu_seqlens=cu)["loss"]
        loss.backward()
        assert abs(float(loss) - float(ref)) < 1e-4, (float(loss), float(ref))
        # the data-parallel reduction AVERAGES over the flattened dp x cp mesh
        for (n, p), (_, pf) in zip(model.named_parameters(), full.named_parameters()):
            gr = p.grad.clone()
            dist.all_reduce(gr)
            gr /= world
            assert torch.allclose(gr, pf.grad, atol=2e-4), (n, (gr - pf.grad).abs().max())
    if rank == 0:
        print(f"{mode} ok")
    dist.destroy_process_group()


if __name__ == "__main__":
    main(sys.argv[1])
