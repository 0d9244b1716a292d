"""Decoder forward/backward on NCCL ranks with the fused-collective projections against the same
model with NCCL collectives around plain GEMMs (``LMMS_B200_FUSED_COMM=0`` semantics): Ulysses
sequence parallelism and sequence-parallel tensor parallelism.  Launched by torchrun."""
import os
import sys

os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import torch
import torch.distributed as dist


def grads_of(model):
    out = {}
    for n, p in model.named_parameters():
        g = p.grad
        out[n] = (g.to_local() if hasattr(g, "to_local") else g).float().clone()
    return out


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from torch.distributed.device_mesh import init_device_mesh

    from lmms_engine_b200.models.decoder_lm import DecoderConfig, DecoderLM
    from lmms_engine_b200.ops import _cuda
    from lmms_engine_b200.parallel import fused_ops
    from lmms_engine_b200.parallel.tensor_parallel import shard_decoder_for_tp

    cfg = DecoderConfig(model_type="qwen2", vocab_size=512, hidden_size=512, intermediate_size=1024, num_hidden_layers=2,
                        num_attention_heads=2 * world, num_key_value_heads=world, head_dim=64, attention_bias=True)
    T = 512 * world
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(0, 512, (T,), generator=g).to(dev)
    cu = torch.tensor([0, 300, 700, T][: 4 if T > 700 else 2] if T > 700 else [0, T], dtype=torch.int32, device=dev)

    def build():
        torch.manual_seed(0)
        return DecoderLM(cfg).to(dev, torch.bfloat16)

    results = {}
    for mode in ("ulysses", "tp"):
        for fused in (False, True):
            os.environ["LMMS_B200_FUSED_COMM"] = "1" if fused else "0"
            fused_ops._CONTEXTS.clear()
            model = build()
            if mode == "ulysses":
                model.sp_group = dist.group.WORLD
            else:
                mesh = init_device_mesh("cuda", (world,), mesh_dim_names=("tp",))
                shard_decoder_for_tp(model, mesh, mesh.get_group())
            losses = []
            for _ in range(2):  # the second pass re-uses every buffer and its counters
                model.zero_grad(set_to_none=True)
                loss = model(input_ids=ids, labels=ids, cu_seqlens=cu)["loss"]
                loss.backward()
                losses.append(float(loss))
            torch.cuda.synchronize()
            _cuda.check_status()
            if fused:
                ctx = fused_ops._CONTEXTS.get(id(dist.group.WORLD if mode == "ulysses" else mesh.get_group()))
                assert ctx is not None and ctx.launches > 0, "the fused kernels did not run"
            results[(mode, fused)] = (losses, grads_of(model))
        (l0, g0), (l1, g1) = results[(mode, False)], results[(mode, True)]
        assert abs(l0[0] - l1[0]) < 2e-2 and abs(l0[1] - l1[1]) < 2e-2, (mode, l0, l1)
        for n in g0:
            scale = max(1.0, g0[n].abs().max().item())
            err = (g0[n] - g1[n]).abs().max().item()
            assert err <= 4e-2 * scale, (mode, n, err, scale)
    dist.barrier()
    if rank == 0:
        print("fused model ok")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
