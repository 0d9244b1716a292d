"""Multi-rank check of the peer-memory runtime, one rank per GPU (launched by torchrun).

1. PeerComm.reduce_to_owner / publish against NCCL reduce / broadcast on the same data.
2. Three optimizer steps of a small decoder with the owner-sharded runtime on PeerComm (buckets
   reduced during the backward pass; reduced only at the step; fp32 gradient buffer) and on
   TorchComm: parameters must agree across ranks and across the implementations.
NVLS is kept off (plain peer loads and stores only)."""
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
    from lmms_engine_b200.models.decoder_lm import DecoderConfig, DecoderLM
    from lmms_engine_b200.ops import _cuda
    from lmms_engine_b200.parallel.owner_sharded import OwnerShardedRuntime, TorchComm
    from lmms_engine_b200.parallel.peer_comm import PeerComm

    comm = PeerComm(None, dev)
    # ---- 1. raw collectives --------------------------------------------------------------
    total = 1 << 20
    chunk = total // world
    ranges = [[(r * chunk, (r + 1) * chunk), (0, 0)] for r in range(world)]
    g = comm.allocate(total, torch.bfloat16, dev)
    torch.manual_seed(100 + rank)
    g.copy_(torch.randn(total, device=dev).to(torch.bfloat16))
    ref = g.clone().float()
    dist.all_reduce(ref)
    comm.reduce_to_owner(g, ranges)
    torch.cuda.synchronize()
    lo, hi = ranges[rank][0]
    err = (g[lo:hi].float() - ref[lo:hi]).abs().max().item()
    assert err < 0.1, err
    comm.publish(g, ranges)
    torch.cuda.synchronize()
    full = g.clone()
    dist.broadcast(full, src=0)
    assert torch.equal(full, g), "replicas differ after publish"
    assert (g.float() - ref).abs().max().item() < 0.1
    _cuda.check_status()

    # ---- 2. training steps: PeerComm vs TorchComm --------------------------------------------
    cfg = DecoderConfig(model_type="qwen2", vocab_size=4096, hidden_size=512, intermediate_size=1408,
                        num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=128)
    results = []
    variants = [("peer, reduce during backward", lambda: comm, True, torch.bfloat16),
                ("peer, reduce at the step", lambda: comm, False, torch.bfloat16),
                ("peer, fp32 gradients", lambda: comm, True, torch.float32),
                ("torch.distributed", lambda: TorchComm(dist.group.WORLD), False, torch.bfloat16)]
    for label, make_comm, armed, grad_dtype in variants:
        torch.manual_seed(0)
        with torch.device(dev):
            model = DecoderLM(cfg).to(torch.bfloat16)
        rt = OwnerShardedRuntime(model, dist.group.WORLD, lr=1e-3, weight_decay=0.01, use_muon=True, device=dev, comm=make_comm(),
                                 grad_dtype=grad_dtype)
        assert rt.overlap == (label.startswith("peer")), label
        torch.manual_seed(7 + rank)
        for step in range(3):
            ids = torch.randint(0, 4096, (1024,), device=dev)
            cu = torch.tensor([0, 300, 1024], dtype=torch.int32, device=dev)
            out = model(input_ids=ids, labels=ids, cu_seqlens=cu)
            if armed:
                rt.arm()
            out["loss"].backward()
            if armed and step == 0:
                assert all(rt._fired), "every bucket should have been reduced by its backward hook"
            rt.step()
        torch.cuda.synchronize()
        _cuda.check_status()
        mine = rt.P.clone()
        other = mine.clone()
        dist.broadcast(other, src=0)
        assert torch.equal(mine, other), "replicas diverged"
        results.append(mine.float())
    diff = max((r - results[-1]).abs().max().item() for r in results[:-1])
    assert diff < 2e-2, diff

    # ---- 3. the buckets reduced during the backward pass hold COMPLETE gradients -----------------
    # (parameters after a step are not bit-reproducible: Muon's norm uses floating-point atomics)
    torch.manual_seed(0)
    with torch.device(dev):
        model = DecoderLM(cfg).to(torch.bfloat16)
    rt = OwnerShardedRuntime(model, dist.group.WORLD, lr=1e-3, use_muon=True, device=dev, comm=comm)
    torch.manual_seed(11 + rank)
    ids = torch.randint(0, 4096, (1024,), device=dev)
    cu = torch.tensor([0, 500, 1024], dtype=torch.int32, device=dev)
    model(input_ids=ids, labels=ids, cu_seqlens=cu)["loss"].backward()  # not armed: local gradients only
    expected = rt.G.clone().float()
    dist.all_reduce(expected)
    rt.G.zero_()
    rt.arm()
    model(input_ids=ids, labels=ids, cu_seqlens=cu)["loss"].backward()
    assert all(rt._fired)
    rt._finish_reduce()
    torch.cuda.synchronize()
    _cuda.check_status()
    for lo, hi in rt.all_ranges[rank]:
        got, want = rt.G[lo:hi].float(), expected[lo:hi]
        err = (got - want).abs().max().item()
        assert err <= 1e-2 * (want.abs().max().item() + 1e-6) + 1e-6, (lo, hi, err)
    comm.barrier()  # peers have finished reading this rank's gradients
    torch.cuda.synchronize()
    if rank == 0:
        print(f"peer runtime ok: world {world}, max param diff peer-vs-nccl {diff:.2e}")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
