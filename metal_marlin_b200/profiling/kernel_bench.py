"""Per-kernel micro-benchmarks at the flagship model's shapes (GLM-4.7-Flash decode), the target of the
``ncu`` captures summarised under ``profiles/``.

    python -m metal_marlin_b200.profiling.kernel_bench --op all --iters 20
    python -m metal_marlin_b200.profiling.kernel_bench --op moe_gate_up --iters 3 --warmup 1      # small: for ncu
    python -m metal_marlin_b200.profiling.kernel_bench --op gemm_32768x2048x5120,bf16gemm_32768x2048x5120,cublas_32768x2048x5120

Every op is timed with CUDA events on the launching stream after warm-up, with a write of a 256 MB buffer
between iterations so the 126 MB L2 is cold, and reported with its algorithmic bytes and the fraction of the
measured copy bandwidth (``MEASURED_PEAKS.json``; 6.65 TB/s fallback).

Parity: the reference's ``benchmarks/`` drivers and ``metal_marlin/profiling/roofline.py:223``.
"""
from __future__ import annotations

import argparse
import json
import os

import torch

from .. import ops
from ..ops import FP4ExpertBank, FP4Weight


def _peak_gbs() -> float:
    here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    p = os.path.join(here, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return float(json.load(f).get("hbm_gbs", 6650.0))
    return 6650.0


def _rand_w(n, k, dev):
    return FP4Weight.from_float(torch.randn(n, k, device=dev) * 0.02, 128)


def build_cases(dev, batch: int, ctx: int, variants: int = 1):
    """Returns ``{name: (fn, algorithmic_bytes)}``.  ``fn(i)`` runs the op on weight set ``i % variants`` so a
    chain of calls streams distinct weights like consecutive layers of a model do."""
    H, R, dr, dn, dv, NH = 2048, 512, 64, 192, 256, 20
    E, I, topk = 64, 1536, 4
    V = max(1, variants)
    bf = lambda *s: (torch.randn(*s, device=dev) * 0.5).to(torch.bfloat16)
    cases = {}
    x = bf(batch, H)
    delta = bf(batch, H)
    nw = torch.ones(H, device=dev, dtype=torch.bfloat16)
    ro = torch.empty_like(x)

    def clones(w):
        return [w] + [FP4Weight(w.qtile.clone(), w.stile.clone(), w.out_features, w.in_features, w.group_size) for _ in range(V - 1)]

    w_qa = clones(_rand_w(768 + 576, H, dev))
    cases["qa_kva_gemv"] = (lambda i=0: ops.linear(x, w_qa[i % V], delta=delta, norm_w=nw, resid_out=ro), w_qa[0].nbytes())
    w_qb = clones(_rand_w(NH * 256, 768, dev))
    a = bf(batch, 1344)
    nq = torch.ones(768, device=dev, dtype=torch.bfloat16)
    cases["q_b_gemv"] = (lambda i=0: ops.linear(a[:, :768], w_qb[i % V], norm_w=nq), w_qb[0].nbytes())
    w_o = clones(_rand_w(H, NH * dv, dev))
    ao = bf(batch, NH * dv)
    cases["o_proj_gemv"] = (lambda i=0: ops.linear(ao, w_o[i % V]), w_o[0].nbytes())
    # MLA prologue / attention / epilogue
    q = bf(batch, NH * (dn + dr))
    kva = bf(batch, R + dr)
    w_ukT = [bf(NH, R, dn) for _ in range(V)]
    w_uv = [bf(NH, dv, R) for _ in range(V)]
    nkv = torch.ones(R, device=dev, dtype=torch.bfloat16)
    bs = 16
    nb = (ctx + bs) // bs + 1
    cache = [bf(batch * nb * bs, R + dr) for _ in range(V)]
    bt = torch.arange(batch * nb, dtype=torch.int32, device=dev).view(batch, nb)
    cl = torch.full((batch,), ctx, dtype=torch.int32, device=dev)
    pos = torch.full((batch,), ctx - 1, dtype=torch.int32, device=dev)
    slots = (bt[:, (ctx - 1) // bs].long() * bs + (ctx - 1) % bs)
    inv = 1.0 / (1e6 ** (torch.arange(0, dr, 2, device=dev).float() / dr))
    qf = torch.empty(batch, NH, R + dr, dtype=torch.bfloat16, device=dev)
    cases["mla_prep"] = (lambda i=0: ops.mla_prep(q, kva, w_ukT[i % V], nkv, pos, inv, slots, qf, cache[i % V], NH, dn, dr, R, 1e-5,
                                                  1.0, True), w_ukT[0].numel() * 2)
    splits = ops.default_splits(batch, 1, ctx, mla_latent=True)
    cases["mla_decode_attn"] = (lambda i=0: ops.paged_attention(qf, cache[i % V], None, bt, cl, Hq=NH, Hkv=1, dqk=R + dr, dv=R,
                                                                block_size=bs, scale=1 / 16.0, splits=splits, w_uv=w_uv[i % V]),
                                batch * ctx * (R + dr) * 2 + w_uv[0].numel() * 2)
    cache8 = []
    for c in cache:       # the same latent rows in an FP8 pool (E4M3 + per-row scale)
        p8 = ops.FP8KV(c.shape[0], (R + dr,), dev)
        p8.store(torch.arange(c.shape[0], device=dev), c.float())
        cache8.append(p8)
    cases["mla_decode_attn_fp8kv"] = (lambda i=0: ops.paged_attention(qf, cache8[i % V], None, bt, cl, Hq=NH, Hkv=1, dqk=R + dr, dv=R,
                                                                      block_size=bs, scale=1 / 16.0, splits=splits, w_uv=w_uv[i % V]),
                                      batch * ctx * (R + dr + 4) + w_uv[0].numel() * 2)
    part_o = torch.empty(batch * NH * splits * R, dtype=torch.float32, device=dev)
    part_ml = torch.empty(batch * NH * splits * 2, dtype=torch.float32, device=dev)
    o_att = torch.empty(batch, NH, dv, dtype=torch.bfloat16, device=dev)
    ops.paged_attention(qf, cache[0], None, bt, cl, Hq=NH, Hkv=1, dqk=R + dr, dv=R, block_size=bs, scale=1 / 16.0, splits=splits,
                        w_uv=w_uv[0], workspace=(part_o, part_ml), out=o_att)          # fills the partials for the merge-only case
    cases["paged_decode_only"] = (lambda i=0: ops.K.mmb200.paged_decode(qf, cache[i % V], None, bt, cl, part_o, part_ml, NH, 1, R + dr, R,
                                                                        bs, splits, 1 / 16.0, 0),
                                  batch * ctx * (R + dr) * 2)
    cases["decode_merge_only"] = (lambda i=0: ops.K.mmb200.decode_merge(part_o, part_ml, w_uv[i % V], o_att, batch, NH, R, dv, splits),
                                  w_uv[0].numel() * 2 + part_o.numel() * 4)
    tiny = bf(batch, H)
    cases["launch_floor_add"] = (lambda i=0: ops.K.mmb200.add(tiny, delta, ro), 3 * tiny.numel() * 2)
    # MoE
    rw = [bf(E, H) for _ in range(V)]
    rb = torch.zeros(E, device=dev)
    ids = [torch.stack([torch.randperm(E, device=dev)[:topk] for _ in range(batch)]).to(torch.int32) for _ in range(V)]
    wts = torch.rand(batch, topk, device=dev)
    cases["moe_router"] = (lambda i=0: ops.moe_router(x, rw[i % V], delta=delta, norm_w=nw, resid_out=ro, bias=rb, topk=topk,
                                                      scoring=1, renorm=True, routed_scale=1.8), rw[0].numel() * 2)
    gu = FP4ExpertBank(torch.randint(-2 ** 31, 2 ** 31 - 1, (E + 1, 2 * I // 16, H // 64, 32, 4), dtype=torch.int32, device=dev),
                       (torch.rand(E + 1, 2 * I // 16, H // 128, 8, 2, device=dev) * 0.01).half(), 2 * I, H, 128)
    dn_b = FP4ExpertBank(torch.randint(-2 ** 31, 2 ** 31 - 1, (E + 1, H // 16, I // 64, 32, 4), dtype=torch.int32, device=dev),
                         (torch.rand(E + 1, H // 16, I // 128, 8, 2, device=dev) * 0.01).half(), H, I, 128)
    slots_per_tok = topk + 1
    active = min(E, batch * topk) + 1
    per_exp_gu = 2 * I * H // 2 + 2 * I * (H // 128) * 2
    per_exp_dn = H * I // 2 + H * (I // 128) * 2
    cases["moe_gate_up"] = (lambda i=0: ops.moe_gate_up(x, gu, ids[i % V], n_shared=1, shared_base=E, norm_w=nw),
                            (batch * slots_per_tok if batch <= 16 else active) * per_exp_gu)
    hi = bf(batch * slots_per_tok, I)
    cases["moe_down"] = (lambda i=0: ops.moe_down(hi, dn_b, ids[i % V], wts, n_shared=1, shared_base=E),
                         (batch * slots_per_tok if batch <= 16 else active) * per_exp_dn)
    cases["moe_forward"] = (lambda i=0: ops.moe_forward(x, gu, dn_b, ids[i % V], wts, n_shared=1, shared_base=E, norm_w=nw),
                            (batch * slots_per_tok if batch <= 16 else active) * (per_exp_gu + per_exp_dn))
    head = bf(154880, H)
    cases["lm_head"] = (lambda i=0: ops.bf16_linear(x, head, delta=delta, norm_w=nw, out_dtype=torch.float32), head.numel() * 2)
    lg = torch.randn(batch, 154880, device=dev)
    cases["argmax"] = (lambda i=0: ops.argmax(lg), lg.numel() * 4)
    # prefill-size GEMMs on the tensor-core path
    xp = bf(4096, H)
    w_gu = _rand_w(2 * I, H, dev)
    cases["gemm_4096x3072x2048"] = (lambda i=0: ops.linear(xp, w_gu), 2.0 * 4096 * 2 * I * H)
    return cases


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", default="all")
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--ctx", type=int, default=4096)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-flush", action="store_true")
    ap.add_argument("--chain", type=int, default=0,
                    help="time a CUDA graph of this many dependent launches of the op on distinct weight sets "
                         "(in-graph cost per launch, as inside a decode step) instead of isolated cold launches")
    ap.add_argument("--grouped-tune", default="",
                    help="wpt,upi,wpt,upi of the expert-sorted streaming MoE launches (gate-up, down); 0 = launcher's choice")
    args = ap.parse_args()
    dev = torch.device("cuda")
    assert ops.native_available()
    if args.grouped_tune:
        ops.GROUPED_GEMV_TUNE[:] = [int(v) for v in args.grouped_tune.split(",")]
    cases = build_cases(dev, args.batch, args.ctx, variants=max(1, args.chain))
    names = list(cases) if args.op == "all" else args.op.split(",")
    for n in names:
        # gemm_<tokens>x<out>x<in>, bf16gemm_... (both operands by TMA) and cublas_... (torch.matmul) for any shape
        kind, _, dims = n.partition("_")
        if n not in cases and kind in ("gemm", "bf16gemm", "cublas") and dims.count("x") == 2:
            M, N, Kd = (int(v) for v in dims.split("x"))
            xq = (torch.randn(M, Kd, device=dev) * 0.5).to(torch.bfloat16)
            wf = torch.randn(N, Kd, device=dev) * 0.02
            if kind == "gemm":
                wq = FP4Weight.from_float(wf, 128)
                cases[n] = (lambda i=0, xq=xq, wq=wq: ops.linear(xq, wq), 2.0 * M * N * Kd)
            elif kind == "bf16gemm":
                wb = wf.to(torch.bfloat16)
                cases[n] = (lambda i=0, xq=xq, wb=wb: ops.bf16_gemm(xq, wb), 2.0 * M * N * Kd)
            else:
                wt = wf.to(torch.bfloat16).t()
                cases[n] = (lambda i=0, xq=xq, wt=wt: torch.matmul(xq, wt), 2.0 * M * N * Kd)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    peak = _peak_gbs()
    out = {}
    for n in names:
        fn, nbytes = cases[n]
        for _ in range(args.warmup):
            fn()
        torch.cuda.synchronize()
        ts = []
        if args.chain > 0:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for i in range(args.chain):
                    fn(i)
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side):
                    for i in range(args.chain):
                        fn(i)
            torch.cuda.current_stream().wait_stream(side)
            graph.replay()
            torch.cuda.synchronize()
            for _ in range(args.iters):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                graph.replay()
                e1.record()
                torch.cuda.synchronize()
                ts.append(e0.elapsed_time(e1) * 1e3 / args.chain)
            ts.sort()
            med = ts[len(ts) // 2]
            gbs = nbytes / med / 1e3
            out[n] = {"us_per_launch_in_graph": round(med, 2), "chain": args.chain, "MB": round(nbytes / 1e6, 3), "GBps": round(gbs, 1)}
            print(n, out[n], flush=True)
            del graph
            continue
        for _ in range(args.iters):
            if not args.no_flush:
                flush.fill_(1)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) * 1e3)
        ts.sort()
        med = ts[len(ts) // 2]
        if n.split("_")[0] in ("gemm", "bf16gemm", "cublas"):
            out[n] = {"us": round(med, 2), "tflops": round(nbytes / med / 1e6, 1)}
        else:
            gbs = nbytes / med / 1e3
            out[n] = {"us": round(med, 2), "MB": round(nbytes / 1e6, 3), "GBps": round(gbs, 1), "frac_of_measured_copy": round(gbs / peak, 3)}
        print(n, out[n], flush=True)
    print(json.dumps({"batch": args.batch, "ctx": args.ctx, "results": out}))


if __name__ == "__main__":
    main()
