"""Peer-memory reduce / publish kernels.  With one GPU the "peers" are separate buffers on
the same device, which exercises the same loads and stores; the multi-rank path with the
epoch barrier runs under torchrun on two GPUs (tests/helpers/peer_two_gpu.py)."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _arr(tensors):
    return (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])


@pytest.mark.parametrize("n", [2, 4, 8])
def test_reduce_to_owner_and_publish_emulated(n):
    from lmms_engine_b200.ops import _cuda
    from lmms_engine_b200.parallel import peer_comm  # noqa: F401  (registers the entry points)

    total, lo, hi = 1 << 16, 4096, 4096 + 3 * 8192
    bufs = [torch.randn(total, device="cuda").to(torch.bfloat16) for _ in range(n)]
    ref = torch.stack([b[lo:hi].float() for b in bufs]).sum(0) / n
    before = [b.clone() for b in bufs]
    arr = _arr(bufs)
    owner = n - 1
    _cuda.call("b200_peer_reduce_bf16", ctypes.addressof(arr), n, owner, lo, hi - lo, 1.0 / n, _cuda.stream())
    torch.cuda.synchronize()
    assert torch.allclose(bufs[owner][lo:hi].float(), ref, atol=2e-2, rtol=2e-2)
    assert torch.equal(bufs[owner][:lo], before[owner][:lo]) and torch.equal(bufs[owner][hi:], before[owner][hi:])
    for r in range(n - 1):
        assert torch.equal(bufs[r], before[r])
    _cuda.call("b200_peer_publish", ctypes.addressof(arr), n, owner, lo * 2, (hi - lo) * 2, _cuda.stream())
    torch.cuda.synchronize()
    for r in range(n - 1):
        assert torch.equal(bufs[r][lo:hi], bufs[owner][lo:hi])
        assert torch.equal(bufs[r][:lo], before[r][:lo])
