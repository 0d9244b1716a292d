"""Multi-rank check and timing of the GEMMs with fused collectives, one rank per GPU (torchrun).
Every op is compared with the same product computed by plain matmuls + NCCL collectives; with
``FUSED_COMM_TIME=1`` each op is also timed (CUDA events, max over ranks) against that baseline
and one JSON line per op is printed by rank 0.  NVLS off, plain peer stores only."""
import json
import os
import sys

os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import torch
import torch.distributed as dist


_BLOCK = None


def timed(fn, iters=10, warm=3):
    """Device time per call.  A few milliseconds of unrelated GEMMs are queued first so that the
    host has enqueued every timed launch before the first one starts (no launch gaps in the span)."""
    global _BLOCK
    if _BLOCK is None:
        _BLOCK = torch.randn(8192, 8192, device="cuda", dtype=torch.bfloat16)
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(6):
        torch.mm(_BLOCK, _BLOCK)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from lmms_engine_b200.ops import _cuda
    from lmms_engine_b200.ops.gemm import gemm
    from lmms_engine_b200.parallel.fused_comm import FusedComm, out_head_route, qkv_head_route, qkv_kb_sources

    big = os.environ.get("FUSED_COMM_TIME") == "1"
    fc = FusedComm(dist.group.WORLD, dev, wait_ms=20000, chunk_bytes=(1 << 30) if big else (64 << 20))
    g = torch.Generator(device="cuda")
    rnd = lambda seed, *shape, scale=1.0: (torch.randn(*shape, device=dev, generator=g.manual_seed(seed)) * scale).to(torch.bfloat16)
    close = lambda a, b, tol=3e-2: (a.float() - b.float()).abs().max().item() <= tol * max(1.0, b.float().abs().max().item())
    report = []

    # sizes: hidden H, ffn F per rank, tokens per rank Ms
    H, F, Ms = (3584, 18944 // world // 64 * 64, 2048) if big else (256, 384, 256)
    # ---- all-gather -> GEMM (column-parallel up projection) --------------------------------------
    x = rnd(10 + rank, Ms, H)
    w_up = rnd(20 + rank, F, H, scale=0.03)
    y, gathered = fc.ag_gemm(x, w_up)
    xg = torch.empty(Ms * world, H, dtype=torch.bfloat16, device=dev)
    dist.all_gather_into_tensor(xg, x)
    torch.cuda.synchronize()
    if not torch.equal(gathered, xg):
        for r in range(world):
            blk, ref = gathered[r * Ms:(r + 1) * Ms], xg[r * Ms:(r + 1) * Ms]
            bad = (blk != ref)
            print(f"[rank {rank}] block {r}: {int(bad.sum())} of {bad.numel()} differ, zeros in block {int((blk == 0).sum())}, "
                  f"bad rows {bad.any(1).nonzero().flatten()[:8].tolist()} flags {fc._buffers['ag'].flags.tolist()}", flush=True)
        raise AssertionError("gathered rows differ")
    assert close(y, xg.float() @ w_up.float().t()), "ag_gemm"
    # the same product with the copy engines moving the rows (side stream + per-source flags)
    for _ in range(3):
        y2, gathered2 = fc.ag_gemm(x, w_up, key="ag_ce", engine="ce")
    torch.cuda.synchronize()
    assert torch.equal(gathered2, xg) and close(y2, xg.float() @ w_up.float().t()), "ag_gemm (copy engines)"
    # ---- GEMM -> reduce-scatter (row-parallel down projection) -----------------------------------
    h = rnd(30 + rank, Ms * world, F, scale=0.5)
    w_dn = rnd(40 + rank, H, F, scale=0.03)
    for _ in range(2):
        z = fc.gemm_rs(h, w_dn)
    full = (h.float() @ w_dn.float().t())
    dist.all_reduce(full)
    torch.cuda.synchronize()
    assert close(z, full[rank * Ms:(rank + 1) * Ms], 4e-2), "gemm_rs"
    # input gradient of the column-parallel layer with the input re-gathered on the side
    dy = rnd(50 + rank, Ms * world, F, scale=0.5)
    dx, xg2 = fc.gemm_rs(dy, w_up, b_mn=True, key="rs_dx", regather=(x, "regather"))
    full = dy.float() @ w_up.float()
    dist.all_reduce(full)
    torch.cuda.synchronize()
    assert torch.equal(xg2, xg) and close(dx, full[rank * Ms:(rank + 1) * Ms], 4e-2), "gemm_rs + regather"
    # ---- Ulysses: QKV projection -> heads, heads -> output projection -----------------------------
    nq, nkv, D = (28, 4, 128) if big else (8, 4, 64)
    if nq % world or not (nkv % world == 0 or world % nkv == 0):
        nq, nkv = 8 * world, world
    Hm = nq * D if not big else H
    Tl = Ms
    xs = rnd(60 + rank, Tl, Hm)
    wqkv = rnd(61, (nq + 2 * nkv) * D, Hm, scale=0.03)  # replicated weights (sequence parallel)
    bqkv = rnd(62, (nq + 2 * nkv) * D)
    route = qkv_head_route(nq, nkv, D, world, dev)
    out = fc.gemm_a2a(xs, wqkv, route, bias=bqkv, key=("qkv", 0))
    ref = (xs.float() @ wqkv.float().t() + bqkv.float()).to(torch.bfloat16)
    from lmms_engine_b200.parallel.sequence_parallel import ulysses

    q_ref, k_ref, v_ref = ulysses.seq_to_head_qkv(ref[:, :nq * D].reshape(Tl, nq, D), ref[:, nq * D:(nq + nkv) * D].reshape(Tl, nkv, D),
                                                  ref[:, (nq + nkv) * D:].reshape(Tl, nkv, D), dist.group.WORLD)
    torch.cuda.synchronize()
    hq_l, hkv_l = nq // world, max(nkv // world, 1)
    got_q = out[:, :hq_l * D].reshape(Tl * world, hq_l, D)
    got_k = out[:, hq_l * D:(hq_l + hkv_l) * D].reshape(Tl * world, hkv_l, D)
    got_v = out[:, (hq_l + hkv_l) * D:].reshape(Tl * world, hkv_l, D)
    assert close(got_q, q_ref) and close(got_k, k_ref) and close(got_v, v_ref), "gemm_a2a"
    # output projection: attention output [T, hq_l*D] per rank -> my tokens, all heads
    ao = rnd(70 + rank, Tl * world, hq_l * D)
    wo = rnd(71, Hm, nq * D, scale=0.03)
    ao_seq = ulysses.head_to_seq(ao.view(Tl * world, hq_l, D), dist.group.WORLD).reshape(Tl, nq * D)
    for eng in ("sm", "ce", "ce"):
        yo, gath = fc.a2a_gemm([(ao, rank * hq_l * D)], wo, nq * D, key="o_" + eng, k_rot=rank * hq_l * D // 64, engine=eng)
        torch.cuda.synchronize()
        assert torch.equal(gath, ao_seq), "a2a gather " + eng
        assert close(yo, ao_seq.float() @ wo.float().t()), "a2a_gemm " + eng
    # input gradient of the output projection: GEMM -> heads
    dyo = rnd(80 + rank, Tl, Hm, scale=0.5)
    oroute = out_head_route(nq, D, world, dev)
    dao = fc.gemm_a2a(dyo, wo, oroute, b_mn=True, key=("dao", 0))
    ref = (dyo.float() @ wo.float()).to(torch.bfloat16)
    dao_ref = ulysses.gather_seq_scatter_heads(ref.view(Tl, nq, D), dist.group.WORLD).reshape(Tl * world, hq_l * D)
    torch.cuda.synchronize()
    assert close(dao, dao_ref), "gemm_a2a (MN-major weight)"
    if nkv % world == 0:
        # input gradient of the QKV projection: three gathered segments, k-blocks waited per source
        dq, dk, dv = rnd(90 + rank, Tl * world, hq_l * D), rnd(91 + rank, Tl * world, hkv_l * D), rnd(92 + rank, Tl * world, hkv_l * D)
        kb = qkv_kb_sources(nq, nkv, D, world, dev)
        seq = lambda t, hh: ulysses.head_to_seq(t.view(Tl * world, hh, D), dist.group.WORLD).reshape(Tl, -1)
        full = torch.cat([seq(dq, hq_l), seq(dk, hkv_l), seq(dv, hkv_l)], 1)
        for eng in ("sm", "ce", "ce"):
            dxs, dqkv = fc.a2a_gemm([(dq, rank * hq_l * D), (dk, nq * D + rank * hkv_l * D), (dv, (nq + nkv) * D + rank * hkv_l * D)],
                                    wqkv, (nq + 2 * nkv) * D, kb_src=kb, b_mn=True, key="dqkv_" + eng, k_rot=rank * hq_l * D // 64,
                                    engine=eng)
            torch.cuda.synchronize()
            assert torch.equal(dqkv, full), "qkv gradient gather " + eng
            assert close(dxs, full.float() @ wqkv.float(), 4e-2), "a2a_gemm (three segments) " + eng
    _cuda.check_status()

    if big:
        def base_ag():
            dist.all_gather_into_tensor(xg, x)
            return gemm(xg, w_up)

        def base_rs():
            p = gemm(h, w_dn)
            o = torch.empty(Ms, H, dtype=torch.bfloat16, device=dev)
            dist.reduce_scatter_tensor(o, p)
            return o

        def base_qkv():
            r = gemm(xs, wqkv, bias=bqkv)
            return ulysses.seq_to_head_qkv(r[:, :nq * D].reshape(Tl, nq, D), r[:, nq * D:(nq + nkv) * D].reshape(Tl, nkv, D),
                                           r[:, (nq + nkv) * D:].reshape(Tl, nkv, D), dist.group.WORLD)

        def base_o():
            s = ulysses.head_to_seq(ao.view(Tl * world, hq_l, D), dist.group.WORLD).reshape(Tl, nq * D)
            return gemm(s, wo)

        cases = [
            ("ag_gemm", lambda: fc.ag_gemm(x, w_up, engine="sm"), base_ag, 2.0 * Ms * world * F * H, (world - 1) * Ms * H * 2),
            ("ag_gemm_ce", lambda: fc.ag_gemm(x, w_up, key="ag_ce", engine="ce"), base_ag, 2.0 * Ms * world * F * H, (world - 1) * Ms * H * 2),
            ("gemm_rs", lambda: fc.gemm_rs(h, w_dn), base_rs, 2.0 * Ms * world * F * H, (world - 1) * Ms * H * 2),
            ("gemm_a2a_qkv", lambda: fc.gemm_a2a(xs, wqkv, route, bias=bqkv, key=("qkv", 0)), base_qkv,
             2.0 * Tl * (nq + 2 * nkv) * D * Hm, (world - 1) / world * Tl * (nq + 2 * nkv) * D * 2),
            ("a2a_gemm_o", lambda: fc.a2a_gemm([(ao, rank * hq_l * D)], wo, nq * D, key="o_sm", k_rot=rank * hq_l * D // 64, engine="sm"), base_o,
             2.0 * Tl * nq * D * Hm, (world - 1) / world * Tl * nq * D * 2),
            ("a2a_gemm_o_ce", lambda: fc.a2a_gemm([(ao, rank * hq_l * D)], wo, nq * D, key="o_ce", k_rot=rank * hq_l * D // 64, engine="ce"), base_o,
             2.0 * Tl * nq * D * Hm, (world - 1) / world * Tl * nq * D * 2),
        ]
        solo = FusedComm(None, dev, wait_ms=20000, chunk_bytes=1 << 30)  # same kernels, no peers
        only = {
            "ag_gemm": (lambda: gemm(xg, w_up), lambda: solo.ag_gemm(xg, w_up)),
            "ag_gemm_ce": (lambda: gemm(xg, w_up), None),
            "gemm_rs": (lambda: gemm(h, w_dn), lambda: solo.gemm_rs(h, w_dn)),
            "gemm_a2a_qkv": (lambda: gemm(xs, wqkv, bias=bqkv), None),
            "a2a_gemm_o": (lambda: gemm(ao_seq, wo), None),
            "a2a_gemm_o_ce": (lambda: gemm(ao_seq, wo), None),
        }
        for name, fused, base, flops, nv_bytes in cases:
            tf, tb = timed(fused), timed(base)
            tg = timed(only[name][0])
            ts = timed(only[name][1]) if only[name][1] is not None else None
            report.append({"op": name, "world": world, "fused_ms": round(tf, 4), "gemm_plus_nccl_ms": round(tb, 4),
                           "gemm_only_ms": round(tg, 4), "fused_single_rank_ms": None if ts is None else round(ts, 4),
                           "speedup": round(tb / tf, 3), "tflops_fused": round(flops / tf / 1e9, 1),
                           "nvlink_out_bytes_per_rank": int(nv_bytes)})
        # timeline of one launch of each pushing kernel (CTA 0, nanoseconds from its start)
        fc.trace = torch.zeros(6, dtype=torch.int64, device=dev)
        for name, fused in (("ag_gemm", cases[0][1]), ("a2a_gemm_o", cases[4][1])):
            for _ in range(3):
                fused()
            torch.cuda.synchronize()
            dist.barrier()
            fused()
            torch.cuda.synchronize()
            tr = fc.trace.tolist()
            print(f"[rank {rank}] {name} timeline us: handshake {(tr[1]-tr[0])/1e3:.1f} first_push {(tr[2]-tr[0])/1e3:.1f} "
                  f"all_push {(tr[3]-tr[0])/1e3:.1f} last_source_seen {(tr[4]-tr[0])/1e3:.1f} end {(tr[5]-tr[0])/1e3:.1f}", flush=True)
        fc.trace = None
        # the exchange by itself: a one-tile-wide GEMM behind the same push (rate = pushed bytes / time)
        w_thin = rnd(99, 256, H, scale=0.03)
        for rows in (512, 2048, 8192):
            xr = rnd(200 + rank, rows, H)
            t_push = timed(lambda: fc.ag_gemm(xr, w_thin, key="thin"))
            t_ref = timed(lambda: gemm(xg[: rows * world] if rows * world <= xg.shape[0] else torch.cat([xg] * (rows * world // xg.shape[0])), w_thin))
            report.append({"op": "push_only_ag", "rows_per_rank": rows, "bytes_to_each_peer": rows * H * 2, "fused_ms": round(t_push, 4),
                           "thin_gemm_only_ms": round(t_ref, 4),
                           "peer_store_gbs": round(rows * H * 2 * (world - 1) / max(t_push - t_ref, 1e-6) / 1e6, 1)})
        _cuda.check_status()
        if rank == 0:
            for r in report:
                print(json.dumps(r))
    dist.barrier()
    if rank == 0:
        print("fused comm ok")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
