"""Expert-parallel dispatch -> grouped expert GEMMs (scatter epilogue) -> combine with the ``ep`` ranks emulated on ONE GPU:
every rank's buffers live on the same device and the ranks are stepped phase by phase (all dispatches, then all expert
passes, then all combines), so no launch ever waits for a later one.  The peer tables of the kernels point into local
memory; the code path, the launches and the bytes stored through the "peer" pointers are the ones of a multi-GPU step, which
makes this the program to put under a profiler (one process, one GPU).

    python -m metal_marlin_b200.profiling.ep_emulated_bench --ep 2 --tokens 1024 --iters 3

Prints one JSON line: CUDA-event time per phase (all ranks together), the bytes the step stores through peer pointers
(token rows out: ``tokens x top-k x hidden`` bf16 + 8 bytes of routing metadata per row; expert rows back: the same rows in
bf16) and the status words.  Numerics of this path: ``tests/test_ep_fused_gpu.py``.
"""
from __future__ import annotations

import argparse
import json

import torch

from .. import ops
from ..ops.weights import FP4ExpertBank
from ..parallel.ep import EPExchange, ExpertParallelMoE


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ep", type=int, default=2)
    ap.add_argument("--tokens", type=int, default=1024, help="tokens held by every emulated rank")
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--inter", type=int, default=1536)
    ap.add_argument("--experts", type=int, default=64)
    ap.add_argument("--topk", type=int, default=4)
    ap.add_argument("--group-size", type=int, default=128)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=2)
    a = ap.parse_args()
    dev = torch.device("cuda")
    torch.manual_seed(0)
    E, H, I, ep, T, k = a.experts, a.hidden, a.inter, a.ep, a.tokens, a.topk
    rnd = lambda *s: torch.randint(-2 ** 31, 2 ** 31 - 1, s, dtype=torch.int32, device=dev)
    sc = lambda *s: (torch.rand(*s, device=dev) * 0.01).half()
    gs = a.group_size
    gu = FP4ExpertBank(rnd(E, 2 * I // 16, H // 64, 32, 4), sc(E, 2 * I // 16, H // gs, 8, 2), 2 * I, H, gs)
    dn = FP4ExpertBank(rnd(E, H // 16, I // 64, 32, 4), sc(E, H // 16, I // gs, 8, 2), H, I, gs)
    nw = torch.ones(H, dtype=torch.bfloat16, device=dev)
    xs = [(torch.randn(T, H, device=dev) * 0.5).to(torch.bfloat16) for _ in range(ep)]
    ids = [torch.stack([torch.randperm(E, device=dev)[:k] for _ in range(T)]).to(torch.int32) for _ in range(ep)]
    wts = [torch.rand(T, k, device=dev) for _ in range(ep)]
    exs = EPExchange.emulated(ep, H, T, k, dev)
    moes = [ExpertParallelMoE(gu, dn, E, 0, r, ep) for r in range(ep)]
    ev = lambda: torch.cuda.Event(enable_timing=True)
    times = {"dispatch": 0.0, "experts": 0.0, "combine": 0.0}
    for it in range(a.warmup + a.iters):
        e = [ev() for _ in range(4)]
        e[0].record()
        states = [moes[r].fused_dispatch(exs[r], xs[r], ids[r], wts[r], norm_w=nw) for r in range(ep)]
        e[1].record()
        for r in range(ep):
            moes[r].fused_experts(exs[r], expected_rows=T * k)
        e[2].record()
        outs = [moes[r].fused_combine(exs[r], states[r]) for r in range(ep)]
        e[3].record()
        torch.cuda.synchronize()
        if it >= a.warmup:
            for j, name in enumerate(times):
                times[name] += e[j].elapsed_time(e[j + 1]) * 1e3 / a.iters
    rows = ep * T * k
    out = {"bench": "ep_emulated", "ep": ep, "tokens_per_rank": T, "hidden": H, "inter": I, "experts": E, "topk": k,
           "us_all_ranks": {n: round(v, 1) for n, v in times.items()}, "us_per_rank_total": round(sum(times.values()) / ep, 1),
           "peer_store_bytes": {"dispatch_rows": rows * H * 2, "dispatch_meta": rows * 8, "return_rows": rows * H * 2},
           "expert_gflop_all_ranks": round(rows * 3 * I * H * 2 / 1e9, 1),
           "exchange_status": [x.check() for x in exs], "status": ops.check_status(dev), "finite": bool(all(torch.isfinite(o.float()).all() for o in outs))}
    print(json.dumps(out))


if __name__ == "__main__":
    main()
