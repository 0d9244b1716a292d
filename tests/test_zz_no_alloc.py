"""The allocation-free RMSNorm backward entry point, called through its exported C symbol.

Some hosts cannot allocate device memory where they call these kernels (a plugin callback of
another runtime, a fixed-budget service): for them the library carries its own scratch.  The
result must equal the regular entry point's, call after call, although every call reuses
the same scratch array."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from lmms_engine_b200 import _native

    lib = _native.lib("elementwise")
    fn = lib.b200_rmsnorm_bwd_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_int, ctypes.c_int, ctypes.c_float, ctypes.c_void_p]
    return fn


def _regular(dy, x, w, rstd):
    from lmms_engine_b200.ops import _cuda

    rows, H = x.shape
    parts = _cuda.fn("b200_num_partials")()
    dx = torch.empty_like(x)
    dw_part = torch.empty((parts, H), dtype=torch.float32, device=x.device)
    dw = torch.empty(H, dtype=torch.float32, device=x.device)
    _cuda.call("b200_norm_bwd", dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), None, None, dx.data_ptr(),
               dw_part.data_ptr(), None, dw.data_ptr(), None, rows, H, 0.0, 0, 0, _cuda.stream())
    return dx, dw


def _case(rows, H, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(rows, H, device="cuda", generator=g).to(torch.bfloat16)
    dy = torch.randn(rows, H, device="cuda", generator=g).to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(H, device="cuda", generator=g)).to(torch.bfloat16)
    rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-6)
    return dy, x, w, rstd


def test_noalloc_matches_regular_entry_point_twice_in_a_row():
    fn = _lib()
    stream = torch.cuda.current_stream().cuda_stream
    # second call is smaller on purpose: stale partial sums of the first call stay in the scratch
    for rows, H, seed in ((1000, 3584, 1), (37, 1024, 2), (513, 128, 3)):
        dy, x, w, rstd = _case(rows, H, seed)
        dx = torch.empty_like(x)
        dw = torch.empty(H, dtype=torch.float32, device="cuda")
        before = torch.cuda.memory_allocated()
        rc = fn(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx.data_ptr(), dw.data_ptr(), rows, H, 0.0, stream)
        assert rc == 0
        assert torch.cuda.memory_allocated() == before
        dx_ref, dw_ref = _regular(dy, x, w, rstd)
        torch.cuda.synchronize()
        assert torch.allclose(dx.float(), dx_ref.float(), atol=2e-2, rtol=2e-2)
        assert torch.allclose(dw, dw_ref, atol=0.3, rtol=3e-2)
        # and against the fp32 formulation
        xf, dyf, wf = x.float(), dy.float(), w.float()
        xh = xf * rstd[:, None]
        gg = dyf * wf
        dx32 = rstd[:, None] * (gg - xh * (gg * xh).mean(-1, keepdim=True))
        assert torch.allclose(dx.float(), dx32, atol=3e-2, rtol=3e-2)
        assert torch.allclose(dw, (dyf * xh).sum(0), atol=0.3, rtol=3e-2)


def test_noalloc_rejects_rows_wider_than_its_scratch():
    fn = _lib()
    dy, x, w, rstd = _case(8, 8192, 4)
    dx = torch.empty_like(x)
    dw = torch.empty(8192, dtype=torch.float32, device="cuda")
    rc = fn(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx.data_ptr(), dw.data_ptr(), 8, 8192, 0.0,
            torch.cuda.current_stream().cuda_stream)
    assert rc == -20
