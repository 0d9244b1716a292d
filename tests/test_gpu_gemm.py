"""tcgen05 GEMM against an fp32 PyTorch reference (all operand layouts and epilogues)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rand(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda", dtype=torch.float32) * scale).to(torch.bfloat16)


def _check(out, ref, tol=2e-2):
    err = (out.float() - ref).abs().max().item()
    den = ref.abs().max().item() + 1e-6
    assert err / den < tol, f"rel err {err / den:.4f}"


SHAPES = [(128, 256, 64), (256, 512, 128), (384, 768, 320), (200, 264, 72), (1024, 3584, 3584), (4096, 2304, 512),
          (77, 40, 24)]


@pytest.fixture(autouse=True, params=["pair", "single"])
def tile_mode(request):
    """Every test runs with 256 x 256 tiles on CTA pairs (the default) and with one-CTA tiles only."""
    from lmms_engine_b200.ops import _cuda

    set_mode = _cuda.fn("b200_gemm_set_pair_mode")
    set_mode(1 if request.param == "pair" else 0)
    yield request.param
    set_mode(1)


@pytest.mark.parametrize("M,N,K", SHAPES)
def test_gemm_nt(M, N, K):
    from lmms_engine_b200.ops import gemm, _cuda

    a, b = _rand(M, K), _rand(N, K)
    out = gemm.gemm(a, b)
    _check(out, a.float() @ b.float().t())
    _cuda.check_status()


@pytest.mark.parametrize("M,N,K", SHAPES[:-1] + [(80, 40, 24)])
def test_gemm_nn_b_mn_major(M, N, K):
    from lmms_engine_b200.ops import gemm, _cuda

    a, b = _rand(M, K), _rand(K, N)
    out = gemm.gemm(a, b, b_mn_major=True)
    _check(out, a.float() @ b.float())
    _cuda.check_status()


@pytest.mark.parametrize("M,N,K", SHAPES[:-1] + [(80, 40, 24)])
def test_gemm_tn_both_mn_major(M, N, K):
    from lmms_engine_b200.ops import gemm, _cuda

    a, b = _rand(K, M), _rand(K, N)
    out = gemm.gemm(a, b, a_mn_major=True, b_mn_major=True)
    _check(out, a.float().t() @ b.float())
    _cuda.check_status()


def test_gemm_bias_beta():
    from lmms_engine_b200.ops import gemm

    M, N, K = 300, 520, 192
    a, b, c, bias = _rand(M, K), _rand(N, K), _rand(M, N), _rand(N)
    out = gemm.gemm(a, b, alpha=0.5, beta=2.0, bias=bias, cin=c)
    _check(out, 0.5 * (a.float() @ b.float().t()) + bias.float() + 2.0 * c.float())


@pytest.mark.parametrize("M,K", [(512, 256), (3584, 1024), (640, 200)])
def test_gemm_symmetric(M, K):
    from lmms_engine_b200.ops import gemm

    x = _rand(M, K, scale=0.1)
    out = gemm.gemm(x, x, symmetric=True)
    ref = x.float() @ x.float().t()
    _check(out, ref)
    assert torch.equal(out, out.t()), "mirrored store must make the result exactly symmetric"
    a = out
    out2 = gemm.gemm(a, a, alpha=2.0, beta=-3.0, cin=a, symmetric=True)
    _check(out2, 2.0 * (a.float() @ a.float().t()) - 3.0 * a.float())


@pytest.mark.parametrize("M,I,K", [(256, 384, 128), (1000, 688, 256), (4096, 18944, 3584)])
def test_gemm_swiglu(M, I, K):
    from lmms_engine_b200.ops import gemm

    x, wg, wu = _rand(M, K), _rand(I, K, scale=0.05), _rand(I, K, scale=0.05)
    h, g, u = gemm.gemm_swiglu(x, wg, wu, store_gu=True)
    gr, ur = x.float() @ wg.float().t(), x.float() @ wu.float().t()
    _check(g, gr)
    _check(u, ur)
    _check(h, torch.nn.functional.silu(g.float()) * u.float(), tol=1e-2)
    h2, _, _ = gemm.gemm_swiglu(x, wg, wu, store_gu=False)
    assert torch.equal(h, h2)


@pytest.mark.parametrize("M,N,K", [(256, 1024, 128), (333, 4104, 256)])
def test_gemm_stats(M, N, K):
    from lmms_engine_b200.ops import gemm

    x, w = _rand(M, K), _rand(N, K, scale=0.2)
    logits, stats = gemm.gemm_stats(x, w)
    ref = x.float() @ w.float().t()
    _check(logits[:, :N], ref)
    lf = logits[:, :N].float()
    mx = stats[..., 0].max(dim=1).values
    lse = mx + torch.log((stats[..., 1] * torch.exp(stats[..., 0] - mx[:, None])).sum(1))
    assert torch.allclose(lse, torch.logsumexp(lf, dim=1), atol=2e-3, rtol=1e-4)


def test_linear_autograd_matches_torch():
    from lmms_engine_b200.ops import gemm

    x = _rand(2, 192, 320).requires_grad_()
    w = _rand(456 // 8 * 8, 320, scale=0.05).requires_grad_()
    b = _rand(456 // 8 * 8).requires_grad_()
    y = gemm.linear(x, w, b)
    dy = _rand(*y.shape)
    y.backward(dy)
    xr, wr, br = (t.detach().float().requires_grad_() for t in (x, w, b))
    yr = torch.nn.functional.linear(xr, wr, br)
    yr.backward(dy.float())
    _check(y, yr.detach())
    _check(x.grad, xr.grad)
    _check(w.grad, wr.grad)
    _check(b.grad, br.grad)
