"""Multi-rank check of the parameter-sharded runtime on peer memory, one rank per GPU (launched by
torchrun): three optimizer steps (the second with two micro-batches) of a small bf16 decoder with
Muon + AdamW must leave the same parameters as the owner-sharded (replicated) runtime, on every
rank.  NVLS is kept off (plain peer loads and stores only)."""
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
    from lmms_engine_b200.parallel.owner_sharded import OwnerShardedRuntime
    from lmms_engine_b200.parallel.param_sharded import ParamShardedRuntime
    from lmms_engine_b200.parallel.peer_comm import PeerComm

    cfg = DecoderConfig(model_type="qwen2", vocab_size=4096, hidden_size=512, intermediate_size=1408,
                        num_hidden_layers=5, num_attention_heads=4, num_key_value_heads=2, head_dim=128)
    results, losses = [], []
    for cls in (OwnerShardedRuntime, ParamShardedRuntime):
        comm = PeerComm(None, dev, barrier_timeout_ms=20000)
        torch.manual_seed(0)
        with torch.device(dev):
            model = DecoderLM(cfg).to(torch.bfloat16)
        model.gradient_checkpointing_enable() if cls is ParamShardedRuntime and hasattr(model, "gradient_checkpointing_enable") else None
        rt = cls(model, dist.group.WORLD, lr=1e-3, weight_decay=0.01, use_muon=True, device=dev, comm=comm)
        torch.manual_seed(7 + rank)
        ls = []
        for step in range(3):
            micro = 2 if step == 1 else 1
            for mb in range(micro):
                ids = torch.randint(0, 4096, (1024,), device=dev)
                cu = torch.tensor([0, 300, 1024], dtype=torch.int32, device=dev)
                out = model(input_ids=ids, labels=ids, cu_seqlens=cu)
                if mb == micro - 1:
                    rt.arm()
                (out["loss"] / micro).backward()
                rt.after_backward()
                ls.append(float(out["loss"].detach()))
            rt.step()
        torch.cuda.synchronize()
        _cuda.check_status()
        if cls is ParamShardedRuntime:
            state = {k: v.detach().float().clone() for k, v in rt.full_state_items()}
        else:
            state = {k: v.detach().float().clone() for k, v in model.named_parameters()}
        results.append(state)
        losses.append(ls)
        del rt, model
    worst = 0.0
    for k, v in results[0].items():
        d = (v - results[1][k]).abs().max().item()
        worst = max(worst, d)
        assert d < 3e-2, (k, d)
    for a, b in zip(*losses):
        assert abs(a - b) < 5e-2, losses
    # every rank holds the same gathered values
    for k, v in results[1].items():
        other = v.clone()
        dist.broadcast(other, src=0)
        assert torch.equal(other, v), k
    if rank == 0:
        print(f"param sharded ok: world {world}, max param diff sharded-vs-replicated {worst:.2e}, losses {losses[1]}")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
