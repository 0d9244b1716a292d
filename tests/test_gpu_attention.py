"""tcgen05 varlen attention (forward and backward) against the fp32 per-document reference."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(lens, Hq, Hkv, D, causal, window=-1, seed=0):
    from lmms_engine_b200.ops import attention, _cuda

    torch.manual_seed(seed)
    T = sum(lens)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device="cuda")
    q = torch.randn(T, Hq, D, device="cuda").to(torch.bfloat16).requires_grad_()
    k = torch.randn(T, Hkv, D, device="cuda").to(torch.bfloat16).requires_grad_()
    v = torch.randn(T, Hkv, D, device="cuda").to(torch.bfloat16).requires_grad_()
    o = attention.varlen_attn(q, k, v, cu, cu, causal=causal, window_size=(window, -1))
    do = torch.randn_like(o)
    o.backward(do)
    _cuda.check_status()
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    orf = attention.varlen_attn_ref(qr, kr, vr, cu, cu, causal=causal, window_left=window)
    orf.backward(do.float())
    assert (o.float() - orf).abs().max().item() < 3e-2
    for name, a, b in (("dq", q.grad, qr.grad), ("dk", k.grad, kr.grad), ("dv", v.grad, vr.grad)):
        err = (a.float() - b).abs().max().item() / (b.abs().max().item() + 1e-6)
        assert err < 3e-2, (name, err)


@pytest.mark.parametrize("lens", [[128], [256, 128], [1, 37, 130, 257, 64], [700, 3, 1025]])
@pytest.mark.parametrize("causal", [True, False])
def test_attn_d128_gqa(lens, causal):
    _case(lens, 4, 2, 128, causal)


def test_attn_d64_mha():
    _case([300, 17, 129], 2, 2, 64, True)


def test_attn_d80_vision_noncausal():
    _case([64, 1024, 400], 4, 4, 80, False)


def test_attn_d72_vision_noncausal():
    _case([256, 100], 2, 2, 72, False)


def test_attn_sliding_window():
    _case([600, 300], 4, 1, 128, True, window=200)


def test_attn_qwen7b_heads():
    _case([2048, 1000], 28, 4, 128, True)


def test_attn_strided_qkv_views():
    from lmms_engine_b200.ops import attention

    T, Hq, Hkv, D = 500, 4, 2, 128
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device="cuda").to(torch.bfloat16)
    q = qkv[:, : Hq * D].view(T, Hq, D)
    k = qkv[:, Hq * D : (Hq + Hkv) * D].view(T, Hkv, D)
    v = qkv[:, (Hq + Hkv) * D :].view(T, Hkv, D)
    cu = torch.tensor([0, 200, 500], dtype=torch.int32, device="cuda")
    o = attention.varlen_attn(q, k, v, cu, cu, causal=True)
    ref = attention.varlen_attn_ref(q.float(), k.float(), v.float(), cu, cu, causal=True)
    assert (o.float() - ref).abs().max().item() < 3e-2


def test_cu_seqlens_past_the_tensor_raise_status_not_a_fault():
    """A cu_seqlens table that reaches past the packed tensor makes the kernel raise its status word and skip
    the document; nothing is written out of bounds and the context stays usable."""
    from lmms_engine_b200.ops import _cuda, attention

    T, H, D = 256, 2, 64
    q = torch.randn(T, H, D, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(T, H, D, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(T, H, D, device="cuda", dtype=torch.bfloat16)
    bad = torch.tensor([0, 128, 384], dtype=torch.int32, device="cuda")  # the second document ends 128 rows past T
    attention.varlen_attn(q, k, v, bad, bad, causal=True)
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="bad shape"):
        _cuda.check_status()
    good = torch.tensor([0, 128, 256], dtype=torch.int32, device="cuda")
    out = attention.varlen_attn(q, k, v, good, good, causal=True)
    ref = attention.varlen_attn_ref(q, k, v, good, good, True, 1.0 / D ** 0.5, -1)
    assert (out.float() - ref.float()).abs().max() < 3e-2
    _cuda.check_status()
    with pytest.raises(NotImplementedError):
        attention.varlen_attn(q, k, v, good, good, causal=False, window_size=(-1, 16))


@pytest.mark.parametrize("causal", [True, False])
def test_queries_shorter_than_keys_bottom_right_aligned(causal):
    """Documents whose keys are a visible prefix followed by the queries' own tokens (the attention splits of the
    unified model): the causal mask is aligned to the END of the keys."""
    from lmms_engine_b200.ops import attention, _cuda

    torch.manual_seed(0)
    lq, lk = [5, 130, 64, 1], [40, 130, 300, 129]
    cu_q = torch.tensor([0] + list(torch.tensor(lq).cumsum(0)), dtype=torch.int32, device="cuda")
    cu_k = torch.tensor([0] + list(torch.tensor(lk).cumsum(0)), dtype=torch.int32, device="cuda")
    q = torch.randn(sum(lq), 4, 64, device="cuda").to(torch.bfloat16).requires_grad_()
    k = torch.randn(sum(lk), 2, 64, device="cuda").to(torch.bfloat16).requires_grad_()
    v = torch.randn(sum(lk), 2, 64, device="cuda").to(torch.bfloat16).requires_grad_()
    o = attention.varlen_attn(q, k, v, cu_q, cu_k, causal=causal)
    do = torch.randn_like(o)
    o.backward(do)
    _cuda.check_status()
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    orf = attention.varlen_attn_ref(qr, kr, vr, cu_q, cu_k, causal=causal)
    orf.backward(do.float())
    assert (o.float() - orf).abs().max().item() < 3e-2
    for name, a, b in (("dq", q.grad, qr.grad), ("dk", k.grad, kr.grad), ("dv", v.grad, vr.grad)):
        err = (a.float() - b).abs().max().item() / (b.abs().max().item() + 1e-6)
        assert err < 3e-2, (name, err)
