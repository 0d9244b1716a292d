"""Per-kernel timings against the library baselines and the measured roofline.

``python -m lmms_engine_b200.ops.microbench [--json OUT]`` times each native kernel at
the shapes of the Qwen2.5-7B training step with CUDA events (3 warm-ups, L2 flushed
between iterations) and prints achieved TFLOP/s or GB/s next to cuBLAS / torch.
"""
from __future__ import annotations

import argparse
import json
import os

import torch


def _flush_l2(buf):
    buf.zero_()


def timeit(fn, iters=10, warmup=3, flush=None):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        if flush is not None:
            _flush_l2(flush)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e))
    ts.sort()
    return ts[len(ts) // 2]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--json", default=None)
    ap.add_argument("--quick", action="store_true")
    ap.add_argument("--only", default=None, help="substring filter on the op name (GEMM shapes only)")
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args()
    from . import gemm, _cuda

    dev = torch.device("cuda")
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
    rows = []

    def rnd(*s):
        return torch.randn(*s, device=dev, dtype=torch.bfloat16) * 0.05

    T = 16384
    shapes = [
        ("qkv_fwd nt", T, 4608, 3584, "nt"),
        ("gate_up_fwd nt", T, 18944, 3584, "nt"),
        ("down_fwd nt", T, 3584, 18944, "nt"),
        ("down_dx nn", T, 18944, 3584, "nn"),
        ("gate_dw tn", 18944, 3584, T, "tn"),
        ("lm_head nt", 8192, 152064, 3584, "nt"),
    ]
    if args.quick:
        shapes = shapes[:2]
    if args.only:
        shapes = [s_ for s_ in shapes if args.only in s_[0]]
    for name, M, N, K, kind in shapes:
        if kind == "nt":
            a, b = rnd(M, K), rnd(N, K)
            mine = lambda: gemm.gemm(a, b)
            lib = lambda: torch.matmul(a, b.t())
        elif kind == "nn":
            a, b = rnd(M, K), rnd(K, N)
            mine = lambda: gemm.gemm(a, b, b_mn_major=True)
            lib = lambda: torch.matmul(a, b)
        else:
            a, b = rnd(K, M), rnd(K, N)
            mine = lambda: gemm.gemm(a, b, a_mn_major=True, b_mn_major=True)
            lib = lambda: torch.matmul(a.t(), b)
        t1 = timeit(mine, iters=args.iters, flush=flush)
        t2 = timeit(lib, iters=args.iters, flush=flush)
        fl = 2.0 * M * N * K
        rows.append({"op": name, "M": M, "N": N, "K": K, "ms": t1, "tflops": fl / t1 / 1e9, "lib_ms": t2,
                     "lib_tflops": fl / t2 / 1e9})
        print(rows[-1], flush=True)
        del a, b
    if args.only == "optim":
        # optimizer passes on one 18944 x 3584 fp32 matrix: the 16-byte kernels against the scalar ones (reached through
        # views that start one element off a 16-byte boundary)
        from . import optim

        n = 18944 * 3584
        for shift, name in ((0, "16-byte"), (1, "scalar")):
            cut = lambda t: t[shift:shift + n]  # noqa: E731
            g, mom, p = cut(torch.randn(n + 8, device=dev)), cut(torch.zeros(n + 8, device=dev)), cut(torch.randn(n + 8, device=dev))
            out, p16 = cut(torch.empty(n + 8, device=dev, dtype=torch.bfloat16)), cut(torch.empty(n + 8, device=dev, dtype=torch.bfloat16))
            m, v, ss = cut(torch.zeros(n + 8, device=dev)), cut(torch.zeros(n + 8, device=dev)), torch.zeros(1, device=dev)
            res = {"op": f"optimizer passes, {name} kernels, {n} elements",
                   "muon_momentum_scale_ms": timeit(lambda: optim.muon_momentum(mom, g, out, ss, beta=0.95, nesterov=True), iters=args.iters, flush=flush),
                   "muon_update_ms": timeit(lambda: optim.muon_update(p, p16, out, lr=0.02, wd=0.1, scale=3.0), iters=args.iters, flush=flush),
                   "sumsq_ms": timeit(lambda: optim.sumsq_(g, ss, False), iters=args.iters, flush=flush),
                   "adamw_ms": timeit(lambda: optim.adamw_step(p, p16, m, v, g, lr=1e-3, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.1, step=1),
                                      iters=args.iters, flush=flush)}
            rows.append(res)
            print(res, flush=True)
        _cuda.check_status()
        return
    if args.only and args.only != "attn":
        _cuda.check_status()
        return
    if args.only in (None, "attn"):
        from . import attention

        for lens in ([8192, 8192], [4096] * 4, [1024] * 16):
            Tq = sum(lens)
            cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=dev)
            q = rnd(Tq, 28, 128).requires_grad_(); k = rnd(Tq, 4, 128).requires_grad_(); v = rnd(Tq, 4, 128).requires_grad_()
            fwd = lambda: attention.varlen_attn(q, k, v, cu, cu, causal=True)
            t_f = timeit(fwd, iters=args.iters, flush=flush)
            o = fwd(); do = torch.randn_like(o)
            res = {"op": f"attn causal 28q/4kv d128 docs {len(lens)}x{lens[0]}", "fwd_ms": t_f}
            fl = sum(4.0 * l * l * 128 * 28 / 2 for l in lens)
            res["fwd_tflops"] = fl / t_f / 1e9
            for impl in ("split", "fused"):
                attention.BACKWARD_IMPL = impl
                def bwd():
                    o2 = attention.varlen_attn(q, k, v, cu, cu, causal=True)
                    o2.backward(do)
                t_fb = timeit(bwd, iters=args.iters, flush=flush)
                res[f"bwd_{impl}_ms"] = t_fb - t_f
                res[f"bwd_{impl}_tflops"] = 2.5 * fl / max(t_fb - t_f, 1e-6) / 1e9
            attention.BACKWARD_IMPL = "split"
            try:
                from flash_attn import flash_attn_varlen_func
                mx = max(lens)
                lib_f = lambda: flash_attn_varlen_func(q, k, v, cu, cu, mx, mx, causal=True)
                t_lf = timeit(lib_f, iters=args.iters, flush=flush)
                def lib_b():
                    flash_attn_varlen_func(q, k, v, cu, cu, mx, mx, causal=True).backward(do)
                t_lfb = timeit(lib_b, iters=args.iters, flush=flush)
                res.update({"lib_fwd_ms": t_lf, "lib_bwd_ms": t_lfb - t_lf})
            except Exception as e:
                res["lib"] = f"unavailable: {type(e).__name__}"
            rows.append(res)
            print(res, flush=True)
    if args.only:
        _cuda.check_status()
        if args.json:
            os.makedirs(os.path.dirname(args.json) or ".", exist_ok=True)
            with open(args.json, "w") as f:
                json.dump(rows, f, indent=1)
        return
    # fused SwiGLU GEMM vs cuBLAS x2 + elementwise
    x, wg, wu = rnd(T, 3584), rnd(18944, 3584), rnd(18944, 3584)
    t1 = timeit(lambda: gemm.gemm_swiglu(x, wg, wu, True), flush=flush)
    def lib_sw():
        g = torch.matmul(x, wg.t()); u = torch.matmul(x, wu.t())
        return torch.nn.functional.silu(g) * u
    t2 = timeit(lib_sw, flush=flush)
    fl = 4.0 * T * 18944 * 3584
    rows.append({"op": "gate_up_swiglu fused", "ms": t1, "tflops": fl / t1 / 1e9, "lib_ms": t2, "lib_tflops": fl / t2 / 1e9})
    print(rows[-1], flush=True)
    # symmetric X X^T (Muon)
    for M, K in ((3584, 18944), (3584, 3584)):
        xx = rnd(M, K)
        t1 = timeit(lambda: gemm.gemm(xx, xx, symmetric=True), flush=flush)
        t2 = timeit(lambda: torch.matmul(xx, xx.t()), flush=flush)
        fl = 2.0 * M * M * K
        rows.append({"op": f"xxt symm {M}x{K}", "ms": t1, "tflops_full_equiv": fl / t1 / 1e9, "lib_ms": t2, "lib_tflops": fl / t2 / 1e9})
        print(rows[-1], flush=True)
    _cuda.check_status()
    if args.json:
        os.makedirs(os.path.dirname(args.json) or ".", exist_ok=True)
        with open(args.json, "w") as f:
            json.dump(rows, f, indent=1)


if __name__ == "__main__":
    main()
