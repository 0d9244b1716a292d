"""Expert parallelism over peer memory against the NCCL all-to-all implementation, one rank per GPU
(torchrun): same MoE decoder, same batches, both dispatchers; losses and gradients must agree.  With
``PEER_EP_TIME=1`` the MoE layer's forward+backward is also timed with both (CUDA events, max over ranks).
NVLS off, plain peer loads and stores."""
import json
import os
import sys

os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import torch
import torch.distributed as dist


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from lmms_engine_b200.models import MoEConfig, MoEDecoderLM
    from lmms_engine_b200.models.moe_lm import SparseMoeBlock
    from lmms_engine_b200.ops import _cuda
    from lmms_engine_b200.parallel.expert_parallel import ExpertParallel
    from lmms_engine_b200.parallel.peer_expert_parallel import PeerExpertParallel

    E = 4 * world
    cfg = MoEConfig(vocab_size=512, hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
                    num_key_value_heads=2, head_dim=64, num_experts=E, num_experts_per_tok=2, moe_intermediate_size=128,
                    router_aux_loss_coef=0.01)
    El = E // world
    peer = PeerExpertParallel(dist.group.WORLD, E, dev)

    def build(kind):
        torch.manual_seed(0)
        m = MoEDecoderLM(cfg).to(dev, torch.bfloat16)
        for blk in m.modules():
            if isinstance(blk, SparseMoeBlock):
                ex = blk.experts
                ex.gate_up_proj = torch.nn.Parameter(ex.gate_up_proj.data[rank * El:(rank + 1) * El].clone())
                ex.down_proj = torch.nn.Parameter(ex.down_proj.data[rank * El:(rank + 1) * El].clone())
                blk.ep = peer if kind == "peer" else ExpertParallel(dist.group.WORLD, E)
        return m

    g = torch.Generator().manual_seed(5 + rank)
    n = 300 + 77 * rank  # ranks hold different token counts
    ids = torch.randint(0, 512, (n,), generator=g).to(dev)
    cu = torch.tensor([0, 100, n], dtype=torch.int32, device=dev)
    res = {}
    for kind in ("nccl", "peer"):
        m = build(kind)
        losses = []
        for _ in range(2):
            m.zero_grad(set_to_none=True)
            out = m(input_ids=ids, labels=ids, cu_seqlens=cu)
            out["loss"].backward()
            losses.append(float(out["loss"]))
        torch.cuda.synchronize()
        _cuda.check_status()
        res[kind] = (losses, {k: p.grad.float().clone() for k, p in m.named_parameters() if p.grad is not None})
    assert peer.launches > 0
    (l0, g0), (l1, g1) = res["nccl"], res["peer"]
    assert abs(l0[0] - l1[0]) < 2e-2 and abs(l0[1] - l1[1]) < 2e-2, (l0, l1)
    assert g0.keys() == g1.keys()
    for k in g0:
        scale = max(1.0, g0[k].abs().max().item())
        err = (g0[k] - g1[k]).abs().max().item()
        assert err <= 4e-2 * scale, (k, err, scale)

    if os.environ.get("PEER_EP_TIME") == "1":
        from lmms_engine_b200.ops import moe as moe_ops

        H, I, k, T = 2048, 768, 8, 8192
        E2 = 16 * world
        El2 = E2 // world
        peer2 = PeerExpertParallel(dist.group.WORLD, E2, dev)
        nccl2 = ExpertParallel(dist.group.WORLD, E2)

        class Ex:
            pass

        ex = Ex()
        gen = torch.Generator(device="cuda").manual_seed(rank)
        ex.gate_up_proj = (torch.randn(El2, 2 * I, H, device=dev, generator=gen) * 0.02).to(torch.bfloat16).requires_grad_(True)
        ex.down_proj = (torch.randn(El2, H, I, device=dev, generator=gen) * 0.02).to(torch.bfloat16).requires_grad_(True)
        x = torch.randn(T, H, device=dev, generator=gen).to(torch.bfloat16).requires_grad_(True)
        logits = torch.randn(T, E2, device=dev, generator=gen)
        _, idx, w, counts = moe_ops.router_topk(logits, k)
        w = w.detach().requires_grad_(True)

        def step(ep):
            y = ep(x, idx, w, counts, ex)
            y.backward(torch.ones_like(y))

        def timed(ep, iters=5):
            for _ in range(2):
                step(ep)
            torch.cuda.synchronize()
            dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(iters):
                step(ep)
            e1.record()
            torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1) / iters], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return t.item()

        t_nccl, t_peer = timed(nccl2), timed(peer2)
        _cuda.check_status()
        if rank == 0:
            print(json.dumps({"op": "moe_layer_fwd_bwd", "world": world, "tokens_per_rank": T, "hidden": H, "experts": E2, "top_k": k,
                              "moe_intermediate": I, "nccl_ms": round(t_nccl, 3), "peer_ms": round(t_peer, 3),
                              "speedup": round(t_nccl / t_peer, 3)}))
    dist.barrier()
    if rank == 0:
        print("peer expert parallel ok")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
