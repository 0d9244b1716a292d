"""GEMMs with fused collective parts on one GPU (a group of one rank runs the same kernel code:
push, arrival waits, scattering epilogue, slot reduction) against fp32 PyTorch products; the
multi-rank runs are in test_gpu_multi.py."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ctx():
    from lmms_engine_b200.parallel.fused_comm import FusedComm

    return FusedComm(None, torch.device("cuda", 0), wait_ms=2000, chunk_bytes=64 << 20)


def _rand(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda") * scale).to(torch.bfloat16)


def _close(got, ref, tol=2e-2):
    err = (got.float() - ref).abs().max().item()
    assert err <= tol * max(1.0, ref.abs().max().item()), err


def test_ag_gemm_single_rank():
    from lmms_engine_b200.ops import _cuda

    fc = _ctx()
    x, w, b = _rand(384, 320), _rand(200, 320, scale=0.05), _rand(200)
    for _ in range(2):  # the second call re-uses the buffer and its counters
        y, gathered = fc.ag_gemm(x, w, bias=b)
        torch.cuda.synchronize()
        _cuda.check_status()
        assert torch.equal(gathered, x)
        _close(y, x.float() @ w.float().t() + b.float())


def test_gemm_rs_single_rank_both_layouts():
    from lmms_engine_b200.ops import _cuda

    fc = _ctx()
    x = _rand(256, 192)
    w_nk, w_kn = _rand(136, 192, scale=0.05), _rand(192, 136, scale=0.05)
    for _ in range(2):
        y = fc.gemm_rs(x, w_nk)
        y2 = fc.gemm_rs(x, w_kn, b_mn=True)
        torch.cuda.synchronize()
        _cuda.check_status()
        _close(y, x.float() @ w_nk.float().t())
        _close(y2, x.float() @ w_kn.float())
    xl = _rand(128, 64)
    y3, g = fc.gemm_rs(x, w_nk, regather=(xl, "regather"))
    torch.cuda.synchronize()
    assert torch.equal(g, xl)
    _close(y3, x.float() @ w_nk.float().t())


def test_gemm_a2a_routes_column_chunks():
    from lmms_engine_b200.ops import _cuda
    from lmms_engine_b200.parallel.fused_comm import HeadRoute, qkv_head_route

    fc = _ctx()
    x, w, b = _rand(200, 128), _rand(512, 128, scale=0.05), _rand(512)
    perm = torch.randperm(8)
    mk = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    route = HeadRoute(mk([0] * 8), mk((perm * 64).tolist()), mk([1] * 8), 512, False)
    out = fc.gemm_a2a(x, w, route, bias=b)
    torch.cuda.synchronize()
    _cuda.check_status()
    ref = x.float() @ w.float().t() + b.float()
    want = torch.empty_like(ref)
    for c in range(8):
        want[:, perm[c] * 64:(perm[c] + 1) * 64] = ref[:, c * 64:(c + 1) * 64]
    _close(out, want)
    r1 = qkv_head_route(4, 2, 128, 1, "cuda")
    assert r1.cols_local == 8 * 128 and r1.chunk_col.tolist() == [i * 64 for i in range(16)]
    r8 = qkv_head_route(8, 2, 128, 4, "cpu")  # kv heads replicated over two ranks each
    assert r8.kv_replicated and r8.chunk_ndst.tolist()[16:] == [2] * 8 and r8.chunk_dst.tolist()[16:20] == [0, 0, 2, 2]


def test_a2a_gemm_three_segments():
    from lmms_engine_b200.ops import _cuda

    fc = _ctx()
    dq, dk, dv = _rand(256, 256), _rand(256, 128), _rand(256, 128)
    w = _rand(512, 320, scale=0.05)  # [K = q|k|v columns, N] read MN-major
    y, gathered = fc.a2a_gemm([(dq, 0), (dk, 256), (dv, 384)], w, 512, b_mn=True)
    torch.cuda.synchronize()
    _cuda.check_status()
    full = torch.cat([dq, dk, dv], 1)
    assert torch.equal(gathered, full)
    _close(y, full.float() @ w.float())


def test_unset_flag_times_out_with_status():
    """A wait that nothing satisfies ends with the status word raised and the context usable."""
    from lmms_engine_b200.ops import _cuda

    fc = _ctx()
    fc.wait_ms = 50
    x, w = _rand(256, 64), _rand(64, 64)
    y = fc.gemm_rs(x, w, key="stuck")
    torch.cuda.synchronize()
    _cuda.check_status()
    fc._buffers["stuck"].n_out += 1000  # as if earlier calls had counted more tiles: this rank would wait for
    fc.world, fc.rank = 2, 0             # a second rank's partial products, which nothing ever sends
    fc._buffers["stuck"].ptrs.append(fc._buffers["stuck"].ptrs[0])
    fc._buffers["stuck"].flag_ptrs.append(fc._buffers["stuck"].flag_ptrs[0])
    fc.gemm_rs(x, w, key="stuck")
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="status"):
        _cuda.check_status()
    assert torch.ones(4, device="cuda").sum().item() == 4.0  # the context still works
