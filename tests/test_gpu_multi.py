"""Multi-GPU checks (skipped with fewer than two visible GPUs): the peer-memory runtime
under torchrun, one rank per GPU."""
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HELPERS = os.path.join(os.path.dirname(__file__), "helpers")


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _torchrun(script, nproc, timeout=600):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), os.path.join(HELPERS, script)]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=timeout)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    return res.stdout


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_peer_runtime_two_gpus():
    out = _torchrun("peer_two_gpu.py", 2)
    assert "peer runtime ok" in out


@pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs four GPUs")
def test_peer_runtime_four_gpus():
    out = _torchrun("peer_two_gpu.py", 4)
    assert "peer runtime ok" in out


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_param_sharded_runtime_two_gpus():
    out = _torchrun("param_sharded_gpu.py", 2)
    assert "param sharded ok" in out


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_fused_comm_gemms_two_gpus():
    out = _torchrun("fused_comm_run.py", 2)
    assert "fused comm ok" in out


@pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs four GPUs")
def test_fused_comm_gemms_four_gpus():
    out = _torchrun("fused_comm_run.py", 4)
    assert "fused comm ok" in out


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_fused_projections_in_decoder_two_gpus():
    out = _torchrun("fused_model_run.py", 2)
    assert "fused model ok" in out


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_peer_expert_parallel_two_gpus():
    out = _torchrun("peer_ep_run.py", 2)
    assert "peer expert parallel ok" in out
