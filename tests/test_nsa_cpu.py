"""Native sparse attention: the vectorised branches against a token-by-token restatement, and the
bagel patch end to end."""
import math

import torch

from lmms_engine_b200.ops import nsa


def _naive(q, k, v, k_cmp, v_cmp, counts, gates, lens, p, scale):
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    G = Hq // Hkv
    out = torch.zeros(T, Hq, D)
    chosen = {}
    at = ac = 0
    per_block = p.block_size // p.kernel_stride
    for L, n in zip(lens, counts):
        nb = (L + p.block_size - 1) // p.block_size
        for i in range(L):
            t = at + i
            vis = [j for j in range(n) if j * p.kernel_stride + p.kernel_size - 1 <= i]
            for hk in range(Hkv):
                score = torch.zeros(nb)
                for g in range(G):
                    h = hk * G + g
                    if vis:
                        s = torch.stack([q[t, h] @ k_cmp[ac + j, hk] for j in vis]) * scale
                        pr = torch.softmax(s, 0)
                        out[t, h] += gates[t, h, 0] * sum(pr[a] * v_cmp[ac + j, hk] for a, j in enumerate(vis))
                        for a, j in enumerate(vis):
                            # window j covers stride-pieces j .. j + kernel/stride - 1
                            for piece in range(j, j + p.kernel_size // p.kernel_stride):
                                if piece // per_block < nb:
                                    score[piece // per_block] += pr[a]
                mine = i // p.block_size
                for b in range(nb):
                    if b > mine:
                        score[b] = -math.inf
                    elif b < p.init_blocks or b > mine - p.local_blocks:
                        score[b] = math.inf
                order = sorted(range(nb), key=lambda b: (-score[b], b))[: p.topk]
                sel = {b for b in order if score[b] > -math.inf}
                chosen[(t, hk)] = sel
                keys = [j for j in range(i + 1) if j // p.block_size in sel]
                win = [j for j in range(i + 1) if j >= i - p.window_size]
                for g in range(G):
                    h = hk * G + g
                    for idx, ks in ((2, keys), (1, win)):
                        s = torch.stack([q[t, h] @ k[at + j, hk] for j in ks]) * scale
                        pr = torch.softmax(s, 0)
                        out[t, h] += gates[t, h, idx] * sum(pr[a] * v[at + j, hk] for a, j in enumerate(ks))
        at += L
        ac += n
    return out, chosen


def test_branches_match_token_by_token_restatement():
    torch.manual_seed(0)
    p = nsa.NSAParams(block_size=8, compress_type="weightedpool", kernel_size=4, kernel_stride=2, topk=3, init_blocks=1,
                      local_blocks=2, window_size=5)
    lens = [37, 3, 20]
    T, Hq, Hkv, D = sum(lens), 4, 2, 8
    cu = torch.tensor([0, 37, 40, 60], dtype=torch.int32)
    q, k, v = torch.randn(T, Hq, D), torch.randn(T, Hkv, D), torch.randn(T, Hkv, D)
    wk = torch.softmax(torch.randn(Hkv, 4), -1)
    pe = 0.1 * torch.randn(Hkv, 4, D)
    k_cmp, counts = nsa.compress(k, wk, cu, 4, 2, pe, "weightedpool")
    v_cmp, _ = nsa.compress(v, None, cu, 4, 2, None, "avgpool")
    assert counts == [17, 0, 9]
    # compression by hand for one window of the last document
    j, base = 3, 40
    want = sum(wk[1, i] * (k[base + j * 2 + i, 1] + pe[1, i]) for i in range(4))
    assert torch.allclose(k_cmp[17 + j, 1], want, atol=1e-6)
    assert torch.allclose(v_cmp[17 + j, 0], v[base + 6: base + 10, 0].mean(0), atol=1e-6)
    gates = torch.sigmoid(torch.randn(T, Hq, 3))
    scale = 1.0 / math.sqrt(D)
    got = nsa.nsa_attention(q, k, v, k_cmp, v_cmp, counts, gates, cu, p, scale)
    want, chosen = _naive(q, k, v, k_cmp, v_cmp, counts, gates, lens, p, scale)
    assert (got - want).abs().max() < 1e-5
    _, idx = nsa.compressed_attention(q, k_cmp, v_cmp, cu, counts, p, scale)
    for (t, hk), sel in chosen.items():
        assert {int(b) for b in idx[t, hk] if b >= 0} == sel, (t, hk)
    # gathered blocks == masked attention, values and gradients
    qg, kg, vg = (t.clone().requires_grad_() for t in (q, k, v))
    qd, kd, vd = (t.clone().requires_grad_() for t in (q, k, v))
    a = nsa.topk_sparse_attention(qg, kg, vg, idx, p.block_size, cu, scale, q_chunk=16, gather=True)
    b = nsa.topk_sparse_attention(qd, kd, vd, idx, p.block_size, cu, scale, gather=False)
    assert (a - b).abs().max() < 1e-5
    probe = torch.randn_like(a)
    (a * probe).sum().backward()
    (b * probe).sum().backward()
    for x, y in ((qg, qd), (kg, kd), (vg, vd)):
        assert (x.grad - y.grad).abs().max() < 1e-4
    # the linear compression starts as the window average
    wl = nsa.compress_weight("linear", Hkv, D, 4)
    k_lin, _ = nsa.compress(k, wl, cu, 4, 2, None, "linear")
    k_avg, _ = nsa.compress(k, None, cu, 4, 2, None, "avgpool")
    assert torch.allclose(k_lin, k_avg, atol=1e-6)


def test_bagel_patch_trains_all_new_parameters():
    from lmms_engine_b200.mapping_func import create_model_from_config
    from lmms_engine_b200.models.monkey_patch import MONKEY_PATCHER

    torch.manual_seed(0)
    model = create_model_from_config("bagel", dict(model_type="bagel", vocab_size=128, hidden_size=32, intermediate_size=64,
                                                   num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=8,
                                                   latent_channels=4, latent_patch_size=2, max_latent_size=8))
    assert MONKEY_PATCHER.apply(model, "bagel", ["nsa"], block_size=8, kernel_size=4, kernel_stride=2, topk=2, window_size=6) == 1
    assert model.config.extra["nsa_config"]["topk"] == 2
    ids = torch.randint(0, 128, (48,))
    cu = torch.tensor([0, 30, 48], dtype=torch.int32)
    out = model(input_ids=ids, labels=ids, cu_seqlens=cu, latent_tokens=torch.randn(6, 16),
                latent_index=torch.arange(10, 16), latent_pos=torch.arange(6), timesteps=torch.full((6,), 0.4))
    out["loss"].backward()
    attn = model.model.layers[0].self_attn
    for name in ("g_proj.weight", "compress_key", "compress_value", "intra_block_pe"):
        g = attn.get_parameter(name).grad
        assert g is not None and g.abs().sum() > 0, name
    assert torch.isfinite(out["loss"])
