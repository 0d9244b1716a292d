"""Parallelism plumbing on CPU/gloo ranks: expert parallel, Ulysses, tensor parallel and the
rank-layout arithmetic, each against the unsharded computation."""
import os
import socket
import subprocess
import sys

import pytest

HELPERS = os.path.join(os.path.dirname(__file__), "helpers")
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def torchrun(script, nproc, *args, timeout=600):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr",
           "127.0.0.1", "--master-port", str(_free_port()), os.path.join(HELPERS, script), *args]
    env = dict(os.environ, OMP_NUM_THREADS="2", CUDA_VISIBLE_DEVICES="")
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=timeout)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    return res.stdout


@pytest.mark.parametrize("world", [2, 4])
def test_expert_parallel_matches_unsharded(world):
    assert "expert parallel ok" in torchrun("ep_run.py", world)


def test_expert_parallel_plans_of_all_moe_families():
    """qwen3_moe, qwen3_5_moe, qwen3_vl_moe, qwen3_omni_moe and aero_realtime (MoE backbone): the registered
    plan shards the experts and the sharded model equals the unsharded one."""
    out = torchrun("ep_plan_run.py", 2)
    assert "expert parallel plans ok: qwen3_moe qwen3_5_moe_text qwen3_vl_moe qwen3_omni_moe_thinker aero_realtime" in out


def test_expert_parallel_plan_with_experts_also_sharded_by_fsdp():
    """4 ranks, ep 2: the experts are split over the ep mesh (dim 0) AND FSDP-sharded over the two replicas (dim 1)."""
    out = torchrun("ep_plan_run.py", 4, "2")
    assert "expert parallel plans ok: qwen3_moe qwen3_vl_moe" in out


def test_rank_layout_arithmetic():
    from lmms_engine_b200.parallel.process_group_manager import RankLayout

    lay = RankLayout(world_size=8, tp=2, cp=2, pp=1, dp=2)
    assert lay.coords(5) == (1, 0, 0, 1)
    assert lay.group_ranks(5, "tp") == [4, 5]
    assert lay.group_ranks(5, "cp") == [5, 7]
    assert lay.group_ranks(5, "dp") == [1, 5]
    assert lay.group_ranks(0, "dp_cp") == [0, 2, 4, 6]
    ep = RankLayout(world_size=8, dp=8, ep=4)
    assert (ep.dp_shard_mod_ep, ep.dp_shard_in_ep) == (2, 4)
    assert ep.group_ranks(5, "ep") == [4, 5, 6, 7]
    with pytest.raises(ValueError):
        RankLayout(world_size=8, dp=8, hsdp_shard=1)
    with pytest.raises(ValueError):
        RankLayout(world_size=8, dp=4, pp=2)
    with pytest.raises(ValueError):
        RankLayout(world_size=8, dp=8, ep=3)


def test_tensor_parallel_matches_unsharded():
    assert "tp ok" in torchrun("tp_run.py", 2, "tp")


@pytest.mark.parametrize("world", [2, 4])
def test_ulysses_matches_unsharded(world):
    # 4 query heads / 1 KV head over 4 ranks also exercises KV-head replication
    assert "ulysses ok" in torchrun("tp_run.py", world, "ulysses")


@pytest.mark.parametrize("mode", ["vl_ulysses", "vl_tp"])
def test_deepstack_features_follow_the_split_token_stream(mode):
    """Deepstack visual features are indexed over the whole sequence; under Ulysses or sequence-parallel tensor
    parallelism every rank adds the rows that fall into its slice."""
    assert f"{mode} ok" in torchrun("tp_run.py", 2, mode)


def test_vision_tower_is_shared_out_over_a_sequence_parallel_group():
    """Four ranks, two images: two ranks run the tower on one image each, two on nothing; features are gathered back and the
    mean of the ranks' gradients is the full model's gradient."""
    assert "vl_ulysses ok" in torchrun("tp_run.py", 4, "vl_ulysses")


def test_ulysses_hybrid_linear_attention_matches_unsharded():
    """Qwen3.5 layers under Ulysses: the linear-attention heads (convolution + delta rule) and the gated-attention heads
    are exchanged around their sequence-wide parts; loss and gradients equal the single-process model."""
    assert "ulysses_hybrid ok" in torchrun("tp_run.py", 2, "ulysses_hybrid")


@pytest.mark.parametrize("world", [2, 4])
def test_linear_attention_state_hand_off_between_ranks(world):
    """Gated-DeltaNet layers under sequence parallelism WITHOUT a head split: every rank keeps its tokens, the recurrent
    state (and the convolution's last rows) pass from rank to rank; loss and gradients equal the unsharded model's, with
    head counts that do not divide the group."""
    assert "ulysses_hybrid_state ok" in torchrun("tp_run.py", world, "ulysses_hybrid_state")


def test_vit_frame_parallel_matches_local_tower():
    assert "vit frame parallel ok" in torchrun("vit_fp_run.py", 3)


def test_expert_layout_computed_on_the_device_equals_the_host_layout():
    """The fixed-capacity layout (no read-back of the count matrix) gives the same destinations and expert-major
    tables as the host layout; an area that is too small withholds the rows that do not fit and raises the status word."""
    import torch

    from lmms_engine_b200.ops import moe as moe_ops
    from lmms_engine_b200.parallel.peer_expert_parallel import PeerExpertParallel

    torch.manual_seed(0)
    ep, E, T, k = 4, 8, 50, 2
    El, TILE = E // ep, moe_ops.TILE
    idx_all = [torch.stack([torch.randperm(E)[:k] for _ in range(T)]) for _ in range(ep)]
    counts_all = torch.stack([torch.bincount(i.flatten(), minlength=E) for i in idx_all]).int()
    for me in range(ep):
        idx = idx_all[me]
        perm = moe_ops.build_permutation(idx.int(), torch.rand(T, k), counts_all[me])
        # host layout, restated: owner r holds its experts in order, each as [source 0 | source 1 | ...] padded to tiles
        P = (counts_all.long() + TILE - 1) // TILE * TILE
        per_expert = P.sum(0)
        rows_per_rank = per_expert.view(ep, El).sum(1)
        cap = int(rows_per_rank.max())
        dest_rank, dest_row, local, _ = PeerExpertParallel.layout_from_counts(counts_all, perm, cap, me, El)
        for t in range(T):
            for j in range(k):
                e = int(idx[t, j])
                row = int(perm.row_of[t, j])
                owner = e // El
                base = int(per_expert[owner * El:e].sum() + P[:me, e].sum())
                assert int(dest_rank[row]) == owner and int(dest_row[row]) == base + (row - int(perm.expert_start[e]))
        assert local.expert_start.tolist() == [0] + per_expert[me * El:(me + 1) * El].cumsum(0).tolist()
        assert local.tile_expert.numel() == cap // TILE
        want_tiles = sum(([i] * int(per_expert[me * El + i] // TILE) for i in range(El)), [])
        assert local.tile_expert.tolist()[: len(want_tiles)] == want_tiles and all(v == -1 for v in local.tile_expert.tolist()[len(want_tiles):])
        # an area one tile too small for the fullest rank
        status = torch.zeros(1, dtype=torch.int32)
        small = cap - TILE
        d_rank, d_row, loc, _ = PeerExpertParallel.layout_from_counts(counts_all, perm, small, me, El, status)
        assert int(status) == 4 and int(d_row.max()) < small and int(loc.expert_start.max()) <= small
