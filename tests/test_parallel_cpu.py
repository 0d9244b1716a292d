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
