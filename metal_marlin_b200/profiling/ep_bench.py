"""Expert-parallel MoE layer with different tokens on every rank: the exchange inside our kernels over NVLink peer memory
(``ExpertParallelMoE.forward_fused``) against the NCCL all-to-all path (``forward_dispatch``) on the same data.

    torchrun --nnodes 1 --nproc-per-node 2 --master-addr 127.0.0.1 -m metal_marlin_b200.profiling.ep_bench --tokens 2048

Defaults are the routed-expert shapes of GLM-4.7-Flash (hidden 2048, expert intermediate 1536, 64 experts, top-4, FP4 group
128).  Timed with CUDA events on every rank after warm-up, max over ranks; the roofline is the slower of the expert FLOPs
at the measured bf16 peak and the bytes every rank must send and receive (token rows out, expert rows back) at the measured
770 GB/s per direction.  Rank 0 prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from .. import ops
from ..ops.weights import FP4ExpertBank
from ..parallel.ep import EPExchange, ExpertParallelMoE
from .roofline import NVLINK_GBS_PER_DIRECTION, load_peaks


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=2048, help="tokens held by every rank")
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--inter", type=int, default=1536)
    ap.add_argument("--experts", type=int, default=64)
    ap.add_argument("--topk", type=int, default=4)
    ap.add_argument("--group-size", type=int, default=128)
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    assert ops.native_available()
    T, H, I, E, k = args.tokens, args.hidden, args.inter, args.experts, args.topk
    torch.manual_seed(3)
    gu = FP4ExpertBank.from_float(torch.randn(E, 2 * I, H, device=dev) * 0.03, args.group_size)
    dn = FP4ExpertBank.from_float(torch.randn(E, H, I, device=dev) * 0.03, args.group_size)
    moe = ExpertParallelMoE(gu, dn, E, 0, rank, world)
    del gu, dn
    torch.manual_seed(10 + rank)
    x = (torch.randn(T, H, device=dev) * 0.5).to(torch.bfloat16)
    ids = torch.stack([torch.randperm(E, device=dev)[:k] for _ in range(T)]).to(torch.int32)
    wts = torch.rand(T, k, device=dev)
    ex = EPExchange.create(H, T, k, dev)
    flush = torch.empty(160 << 20, dtype=torch.uint8, device=dev)

    def timed(fn):
        for _ in range(3):
            fn()
        ts = []
        for _ in range(args.iters):
            flush.zero_()                    # L2 flushed between timed iterations
            torch.cuda.synchronize()
            dist.barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        t = torch.tensor([sorted(ts)[len(ts) // 2]], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    out_f = moe.forward_fused(ex, x, ids, wts)
    out_n = moe.forward_dispatch(x, ids, wts)
    err = float((out_f.float() - out_n.float()).abs().max() / out_n.float().abs().max())
    ms_fused = timed(lambda: moe.forward_fused(ex, x, ids, wts))
    ms_nccl = timed(lambda: moe.forward_dispatch(x, ids, wts))
    status = ex.check()
    peaks = load_peaks()
    flops = 2.0 * T * k * (2 * I * H + H * I)                    # per rank on average (balanced routing)
    remote = T * k * (world - 1) / world                         # rows that leave the rank (and as many come back)
    link_bytes = remote * H * 2
    t_flops = flops / (peaks["bf16_tflops"] * 1e12) * 1e3
    t_link = link_bytes / (NVLINK_GBS_PER_DIRECTION * 1e9) * 1e3  # out and back use the link one after the other
    roof = max(t_flops, 2 * t_link)
    if rank == 0:
        print(json.dumps({"bench": "ep_moe_layer", "ep": world, "tokens_per_rank": T, "hidden": H, "inter": I, "experts": E, "topk": k,
                          "ms_fused_peer_memory": round(ms_fused, 4), "ms_nccl_all_to_all": round(ms_nccl, 4),
                          "speedup": round(ms_nccl / ms_fused, 3), "rel_diff_fused_vs_nccl": err, "exchange_status": status,
                          "roofline_ms": round(roof, 4), "frac_of_roofline_of_measured": round(roof / ms_fused, 3),
                          "flops_ms_at_measured_peak": round(t_flops, 4), "link_ms_one_way_at_770GBs": round(t_link, 4),
                          "timing": "cuda events, median of iters, max over ranks, L2 flushed"}), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
