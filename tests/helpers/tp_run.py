"""Tensor-parallel (sequence-parallel flavour) and Ulysses checks on CPU/gloo ranks against
the unsharded model: same loss, same gradients."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import torch
import torch.distributed as dist


def main(mode):
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    from torch.distributed.device_mesh import init_device_mesh

    from lmms_engine_b200.models.decoder_lm import DecoderConfig, DecoderLM
    from lmms_engine_b200.parallel import tp_ops
    from lmms_engine_b200.parallel.tensor_parallel import shard_decoder_for_tp

    cfg = DecoderConfig(model_type="qwen3", vocab_size=256, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                        num_attention_heads=4, num_key_value_heads=2 if mode == "tp" else 1, head_dim=16)
    build = DecoderLM
    if mode == "ulysses_hybrid":
        # Gated-DeltaNet + gated-attention hybrid: both layer kinds trade the sequence split for a head split
        from lmms_engine_b200.models.qwen3_5 import Qwen35Config, Qwen35LM

        cfg = Qwen35Config(vocab_size=256, hidden_size=64, intermediate_size=128, num_hidden_layers=4, num_attention_heads=4,
                           num_key_value_heads=2, head_dim=16, linear_conv_kernel_dim=4, linear_key_head_dim=16,
                           linear_value_head_dim=16, linear_num_key_heads=2, linear_num_value_heads=4, partial_rotary_factor=0.5)
        build = Qwen35LM
    torch.manual_seed(0)
    full = build(cfg)
    torch.manual_seed(0)
    model = build(cfg)
    if mode == "ulysses_hybrid":
        with torch.no_grad():  # zero-centred norm scales and unit decay parameters would hide mistakes
            for m_ in (full, model):
                g_ = torch.Generator().manual_seed(7)
                for p_ in m_.parameters():
                    if p_.dim() == 1:
                        p_.copy_(0.5 * torch.rand(p_.shape, generator=g_))
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(0, 256, (91,), generator=g)  # not a multiple of the group size: exercises padding
    cu = torch.tensor([0, 40, 91], dtype=torch.int32)
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
