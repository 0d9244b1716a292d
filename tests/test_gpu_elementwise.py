"""Native bandwidth-bound kernels against fp32 PyTorch references."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rand(*shape, scale=1.0, dtype=torch.bfloat16):
    return (torch.randn(*shape, device="cuda", dtype=torch.float32) * scale).to(dtype)


def _close(a, b, atol=2e-2, rtol=2e-2):
    assert torch.allclose(a.float(), b.float(), atol=atol, rtol=rtol), (a.float() - b.float()).abs().max().item()


@pytest.mark.parametrize("rows,H", [(37, 256), (513, 1024), (300, 3584), (64, 4096), (9, 8192), (1000, 128), (70001, 128), (333, 64), (5003, 256)])
def test_rmsnorm_fwd_bwd(rows, H):
    from lmms_engine_b200.ops import norm

    x = _rand(rows, H).requires_grad_()
    w = (1 + 0.1 * _rand(H).float()).to(torch.bfloat16).requires_grad_()
    y = norm.rmsnorm(x, w, 1e-6)
    dy = _rand(rows, H)
    y.backward(dy)
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    yr = xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + 1e-6) * wr
    yr.backward(dy.float())
    _close(y, yr)
    _close(x.grad, xr.grad)
    _close(w.grad, wr.grad, atol=0.3, rtol=3e-2)


def test_rmsnorm_residual():
    from lmms_engine_b200.ops import norm

    rows, H = 257, 3584
    x, r = _rand(rows, H).requires_grad_(), _rand(rows, H).requires_grad_()
    w = (1 + 0.1 * _rand(H).float()).to(torch.bfloat16).requires_grad_()
    y, s = norm.rmsnorm(x, w, 1e-6, residual=r)
    dy, ds = _rand(rows, H), _rand(rows, H)
    (y * dy).sum().backward(retain_graph=True)
    gx_only_y = x.grad.clone()
    x.grad = None
    r.grad = None
    w.grad = None
    ((y * dy).sum() + (s * ds).sum()).backward()
    xr, rr, wr = (t.detach().float().requires_grad_() for t in (x, r, w))
    sr = (xr + rr).to(torch.bfloat16).float() + 0 * (xr + rr)
    sr = xr + rr
    yr = sr * torch.rsqrt(sr.pow(2).mean(-1, keepdim=True) + 1e-6) * wr
    ((yr * dy.float()).sum() + (sr * ds.float()).sum()).backward()
    _close(s, sr)
    _close(y, yr, atol=4e-2)
    _close(x.grad, xr.grad, atol=4e-2)
    _close(r.grad, rr.grad, atol=4e-2)
    assert not torch.equal(gx_only_y, x.grad)


def test_layernorm():
    from lmms_engine_b200.ops import norm

    rows, H = 333, 1152
    x = _rand(rows, H).requires_grad_()
    w, b = (1 + 0.1 * _rand(H).float()).to(torch.bfloat16).requires_grad_(), _rand(H, scale=0.1).requires_grad_()
    y = norm.layernorm(x, w, b, 1e-6)
    dy = _rand(rows, H)
    y.backward(dy)
    xr, wr, br = (t.detach().float().requires_grad_() for t in (x, w, b))
    yr = torch.nn.functional.layer_norm(xr, (H,), wr, br, 1e-6)
    yr.backward(dy.float())
    _close(y, yr)
    _close(x.grad, xr.grad)
    _close(w.grad, wr.grad, atol=0.3, rtol=3e-2)
    _close(b.grad, br.grad, atol=0.3, rtol=3e-2)


@pytest.mark.parametrize("mode,sections", [(0, (0, 0, 0)), (1, (16, 24, 24)), (2, (24, 20, 20))])
def test_rope_table_and_apply(mode, sections):
    from lmms_engine_b200.ops import rope

    T, Hn, D = 777, 6, 128
    pos = torch.randint(0, 5000, (3, T), device="cuda")
    invf = rope.inv_freq(D, 1e6, device="cuda")
    cos, sin = rope.rope_table(pos, invf, mode, sections)
    cr, sr = rope.rope_table_ref(pos, invf, mode, sections)
    _close(cos, cr, atol=2e-3, rtol=0)
    _close(sin, sr, atol=2e-3, rtol=0)
    x = _rand(T, Hn, D).requires_grad_()
    y = rope.rope_apply(x, cos, sin)
    dy = _rand(T, Hn, D)
    y.backward(dy)
    xr = x.detach().float().requires_grad_()
    yr = rope.rope_apply_ref(xr, cr, sr)
    yr.backward(dy.float())
    _close(y, yr)
    _close(x.grad, xr.grad)


def test_rope_strided_view():
    from lmms_engine_b200.ops import rope

    T, Hq, Hkv, D = 130, 4, 2, 128
    qkv = _rand(T, (Hq + 2 * Hkv) * D)
    q = qkv[:, : Hq * D].view(T, Hq, D)
    pos = torch.arange(T, device="cuda")
    cos, sin = rope.rope_table(pos, rope.inv_freq(D, 1e4, device="cuda"))
    y = rope.rope_apply(q, cos, sin)
    _close(y, rope.rope_apply_ref(q.float(), cos, sin))


def test_swiglu():
    from lmms_engine_b200.ops import swiglu

    g, u = _rand(300, 18944).requires_grad_(), _rand(300, 18944).requires_grad_()
    h = swiglu.swiglu(g, u)
    dh = _rand(300, 18944)
    h.backward(dh)
    gr, ur = g.detach().float().requires_grad_(), u.detach().float().requires_grad_()
    hr = torch.nn.functional.silu(gr) * ur
    hr.backward(dh.float())
    _close(h, hr)
    _close(g.grad, gr.grad)
    _close(u.grad, ur.grad)


def test_swiglu_mlp_matches_unfused():
    from lmms_engine_b200.ops import swiglu

    T, H, I = 384, 256, 688
    x = _rand(T, H).requires_grad_()
    wg, wu, wd = (_rand(I, H, scale=0.06).requires_grad_(), _rand(I, H, scale=0.06).requires_grad_(),
                  _rand(H, I, scale=0.04).requires_grad_())
    y = swiglu.swiglu_mlp(x, wg, wu, wd)
    dy = _rand(T, H)
    y.backward(dy)
    ref = [t.detach().float().requires_grad_() for t in (x, wg, wu, wd)]
    lin = torch.nn.functional.linear
    yr = lin(torch.nn.functional.silu(lin(ref[0], ref[1])) * lin(ref[0], ref[2]), ref[3])
    yr.backward(dy.float())
    _close(y, yr, atol=5e-2, rtol=5e-2)
    for a, b in zip((x, wg, wu, wd), ref):
        err = (a.grad.float() - b.grad).abs().max() / (b.grad.abs().max() + 1e-6)
        assert err < 3e-2, err


@pytest.mark.parametrize("gdtype", [torch.bfloat16, torch.float32])
def test_adamw_matches_torch(gdtype):
    from lmms_engine_b200.ops import optim

    n = 1_000_003
    p = torch.randn(n, device="cuda")
    ref = p.clone().requires_grad_()
    opt = torch.optim.AdamW([ref], lr=1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    p16 = p.to(torch.bfloat16)
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    for step in range(1, 4):
        g = torch.randn(n, device="cuda").to(gdtype)
        ref.grad = g.float()
        opt.step()
        optim.adamw_step(p, p16, m, v, g, lr=1e-3, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.1, step=step)
    assert torch.allclose(p, ref.detach(), atol=1e-5, rtol=1e-5)
    assert torch.equal(p16, p.to(torch.bfloat16))


def test_gradnorm_clip_skip():
    from lmms_engine_b200.ops import optim

    g1, g2 = torch.randn(100_001, device="cuda"), _rand(77_777)
    ss = torch.zeros(1, device="cuda")
    optim.sumsq_(g1, ss, False)
    optim.sumsq_(g2, ss, True)
    ref = (g1.double().pow(2).sum() + g2.double().pow(2).sum()).sqrt()
    norm, coef, skip = torch.zeros(1, device="cuda"), torch.zeros(1, device="cuda"), torch.zeros(1, dtype=torch.int32, device="cuda")
    optim.clip_coef(ss, norm, coef, skip, 1.0)
    assert abs(norm.item() - ref.item()) / ref.item() < 1e-5
    assert abs(coef.item() - 1.0 / (ref.item() + 1e-6)) < 1e-6 and skip.item() == 0
    g1c = g1.clone()
    optim.scale_(g1c, coef)
    assert torch.allclose(g1c, g1 * coef.item())
    g1[5] = float("inf")
    optim.sumsq_(g1, ss, False)
    optim.clip_coef(ss, norm, coef, skip, 1.0)
    assert skip.item() == 1
    p = torch.ones(10, device="cuda")
    q = p.clone()
    optim.adamw_step(p, None, torch.zeros_like(p), torch.zeros_like(p), torch.ones_like(p), lr=0.1, beta1=0.9,
                     beta2=0.99, eps=1e-8, wd=0.0, step=1, gscale=coef, skip=skip)
    assert torch.equal(p, q), "update must be skipped on a non-finite norm"


def test_muon_kernels_and_ema():
    from lmms_engine_b200.ops import optim

    n = 512 * 384
    g = _rand(n)
    mom = torch.zeros(n, device="cuda")
    out = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    ss = torch.zeros(1, device="cuda")
    optim.muon_momentum(mom, g, out, ss, beta=0.95, nesterov=True)
    mref = 0.05 * g.float()
    u = g.float() + 0.95 * (mref - g.float())
    assert torch.allclose(mom, mref, atol=1e-6)
    _close(out, u / (u.norm() + 1e-7), atol=1e-4, rtol=2e-2)
    p = torch.randn(n, device="cuda")
    p0 = p.clone()
    p16 = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    optim.muon_update(p, p16, out, lr=0.02, wd=0.1, scale=3.0)
    assert torch.allclose(p, p0 * (1 - 0.002) - 0.06 * out.float(), atol=1e-6)
    ema = torch.zeros(n, device="cuda")
    optim.ema_update(ema, p16, 0.9)
    assert torch.allclose(ema, 0.1 * p16.float(), atol=1e-6)


def test_muon_momentum_fp32_gradient_vector_and_scalar_paths():
    """fp32 gradients (what the native runtimes hold): whole matrices take the 16-byte kernels, an odd length or an
    unaligned view the scalar ones; both agree with the formula and with each other element for element."""
    from lmms_engine_b200.ops import optim

    torch.manual_seed(0)
    for n, shift in ((384 * 256, 0), (384 * 256 + 3, 0), (384 * 256, 1)):
        big_g = torch.randn(n + 8, device="cuda")
        g = big_g[shift:shift + n]
        mom = torch.zeros(n + 8, device="cuda")[shift:shift + n]
        out = torch.empty(n + 8, device="cuda", dtype=torch.bfloat16)[shift:shift + n]
        ss = torch.zeros(1, device="cuda")
        optim.muon_momentum(mom, g, out, ss, beta=0.9, nesterov=True)
        mref = 0.1 * g
        u = g + 0.9 * (mref - g)
        assert torch.allclose(mom, mref, atol=1e-6)
        want = (u.to(torch.bfloat16).float() / (u.norm() + 1e-7)).to(torch.bfloat16)
        assert (out.float() - want.float()).abs().max() <= 2 ** -8 * want.float().abs().max()
        assert abs(float(ss) - float(u.double().pow(2).sum())) < 1e-3 * float(ss)
        p = torch.randn(n + 8, device="cuda")[shift:shift + n]
        p0 = p.clone()
        p16 = torch.empty(n + 8, device="cuda", dtype=torch.bfloat16)[shift:shift + n]
        optim.muon_update(p, p16, out, lr=0.02, wd=0.1, scale=3.0)
        assert torch.allclose(p, p0 * (1 - 0.002) - 0.06 * out.float(), atol=1e-6) and torch.equal(p16, p.to(torch.bfloat16))
        ss2 = torch.zeros(1, device="cuda")
        optim.sumsq_(g, ss2, False)
        assert abs(float(ss2) - float(g.double().pow(2).sum())) < 1e-5 * float(ss2)


def test_gather_scatter_rows():
    from lmms_engine_b200.ops import index

    src = _rand(1000, 256).requires_grad_()
    idx = torch.randperm(1000, device="cuda")[:400]
    idx[7] = -1
    out = index.gather_rows(src, idx)
    ref = src.detach()[idx.clamp(min=0)].clone()
    ref[7] = 0
    assert torch.equal(out, ref)
    out.backward(torch.ones_like(out))
    assert src.grad.float().sum().item() == 399 * 256
    base = _rand(1000, 256)
    rows = _rand(400, 256)
    sc = index.scatter_rows(base, rows, idx, add=True)
    ref = base.clone().float()
    keep = idx >= 0
    ref[idx[keep]] += rows[keep].float()
    _close(sc, ref)


@pytest.mark.parametrize("reduction", ["mean", "sum", "none"])
def test_fused_linear_cross_entropy(reduction):
    from lmms_engine_b200.ops import cross_entropy as ce

    T, H, V = 700, 256, 4104
    h = _rand(T, H).requires_grad_()
    w = _rand(V, H, scale=0.05).requires_grad_()
    labels = torch.randint(0, V, (T,), device="cuda")
    labels[::7] = -100
    loss = ce.fused_linear_cross_entropy(h, w, labels, reduction, chunk_rows=256)
    hr, wr = h.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    lr_ = ce.flce_ref(hr, wr, labels, reduction)
    if reduction == "none":
        gr = torch.rand(T, device="cuda")
        (loss * gr).sum().backward()
        (lr_ * gr).sum().backward()
    else:
        (loss * 0.5).backward()
        (lr_ * 0.5).backward()
    _close(loss, lr_, atol=2e-2, rtol=1e-2)
    for a, b in ((h.grad, hr.grad), (w.grad, wr.grad)):
        err = (a.float() - b).abs().max() / (b.abs().max() + 1e-9)
        assert err < 3e-2, err


def test_plucker_rays_match_reference_formulation():
    from lmms_engine_b200.ops import camera

    B, V, H, W = 2, 5, 48, 84
    K = torch.tensor([400.0, 420.0, W / 2, H / 2], device="cuda").repeat(B, V, 1) * (1 + 0.1 * torch.rand(B, V, 4, device="cuda"))
    rot = torch.linalg.qr(torch.randn(B, V, 3, 3, device="cuda")).Q
    c2w = torch.eye(4, device="cuda").repeat(B, V, 1, 1)
    c2w[..., :3, :3] = rot
    c2w[..., :3, 3] = torch.randn(B, V, 3, device="cuda")
    out = camera.plucker_rays(K, c2w, H, W)
    ref = camera.plucker_rays_ref(K.cpu(), c2w.cpu(), H, W)
    assert torch.allclose(out.cpu(), ref, atol=1e-4, rtol=1e-4)
    cf = camera.plucker_rays(K, c2w, H, W, channels_first=True)
    assert torch.equal(cf, out.permute(0, 1, 4, 2, 3))


def test_newton_schulz_graph_replay_equals_eager_and_reports_time():
    """Small matrices run their Newton-Schulz chain from a captured CUDA graph: same result as the eager chain,
    replay after replay; with ``MUON_GRAPH_TIME`` set the two are timed on a launch-bound size."""
    import os

    from lmms_engine_b200.ops import muon

    torch.manual_seed(0)
    work = {}
    for shape in ((256, 512), (768, 256)):
        for trial in range(3):
            x = torch.randn(shape, device="cuda", dtype=torch.bfloat16)
            x = x / x.float().norm()
            want = muon.newton_schulz(x.clone(), 5, {}).clone()
            got = muon.orthogonalize(x.clone(), 5, work)
            assert ("graph", shape, 5, 0) in work
            assert torch.equal(got, want), (shape, trial)
    big = torch.randn(4096, 256, device="cuda", dtype=torch.bfloat16)
    muon.orthogonalize(big / big.float().norm(), 5, work)
    assert ("graph", (4096, 256), 5, 0) not in work  # large matrices stay eager
    if os.environ.get("MUON_GRAPH_TIME"):
        x = torch.randn(1152, 1152, device="cuda", dtype=torch.bfloat16)
        x = x / x.float().norm()
        for name, fn in (("eager", lambda: muon.newton_schulz(x.clone(), 5, work)), ("graph", lambda: muon.orthogonalize(x, 5, work))):
            for it in range(3):
                if it == 1:
                    torch.cuda.synchronize()
                    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    a.record()
                for _ in range(50):
                    fn()
            b.record()
            torch.cuda.synchronize()
            print(f"MUON_GRAPH_TIME {name}: {a.elapsed_time(b) / 100 * 1000:.1f} us per 1152 x 1152 chain (15 products)", flush=True)
