"""Expert-parallel check on CPU/gloo ranks: a small MoE decoder with ep = world must give
the same loss and the same gradients as the unsharded model on the concatenated batch."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import torch
import torch.distributed as dist


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    from lmms_engine_b200.models import MoEConfig, MoEDecoderLM
    from lmms_engine_b200.parallel.expert_parallel import ExpertParallel
    from lmms_engine_b200.models.moe_lm import SparseMoeBlock

    cfg = MoEConfig(vocab_size=256, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                    num_key_value_heads=2, head_dim=16, num_experts=8, num_experts_per_tok=2, moe_intermediate_size=32,
                    router_aux_loss_coef=0.0)
    torch.manual_seed(0)
    full = MoEDecoderLM(cfg)
    torch.manual_seed(0)
    model = MoEDecoderLM(cfg)
    El = cfg.num_experts // world
    for blk in model.modules():
        if isinstance(blk, SparseMoeBlock):
            ex = blk.experts
            ex.gate_up_proj = torch.nn.Parameter(ex.gate_up_proj.data[rank * El:(rank + 1) * El].clone())
            ex.down_proj = torch.nn.Parameter(ex.down_proj.data[rank * El:(rank + 1) * El].clone())
            blk.ep = ExpertParallel(dist.group.WORLD, cfg.num_experts)
    g = torch.Generator().manual_seed(5)
    batches = [torch.randint(0, 256, (70 + 13 * r,), generator=g) for r in range(world)]
    cus = [torch.tensor([0, 30, b.numel()], dtype=torch.int32) for b in batches]
    out = model(input_ids=batches[rank], labels=batches[rank], cu_seqlens=cus[rank])
    out["loss"].backward()
    # reference: every rank evaluates all batches on the full model
    ref_losses = []
    for b, cu in zip(batches, cus):
        o = full(input_ids=b, labels=b, cu_seqlens=cu)
        o["loss"].backward()
        ref_losses.append(o["loss"].detach())
    assert abs(float(out["loss"]) - float(ref_losses[rank])) < 1e-4, (float(out["loss"]), float(ref_losses[rank]))
    # expert grads: local shard of the sum over ranks' batches
    for (n, p), (_, pf) in zip(model.named_parameters(), full.named_parameters()):
        if "experts" in n:
            ref = pf.grad[rank * El:(rank + 1) * El]
            assert torch.allclose(p.grad, ref, atol=1e-4), n
    # a dense (replicated) parameter: sum of local grads over ranks equals the reference
    pg = model.model.layers[0].self_attn.q_proj.weight.grad.clone()
    dist.all_reduce(pg)
    assert torch.allclose(pg, full.model.layers[0].self_attn.q_proj.weight.grad, atol=1e-4)
    if rank == 0:
        print("expert parallel ok")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
