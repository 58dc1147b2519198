"""Causal prefill attention of one sequence: the tcgen05 kernel (``csrc/attention_fmha_sm100.cu``) against the mma.sync
kernel (``csrc/attention_prefill.cu``) on the same tensors.

    python -m metal_marlin_b200.profiling.fmha_bench --tokens 4096 --heads 20 --dim 256

CUDA events after warm-up; FLOPs counted for the causal half (4 * t^2 / 2 * heads * dim).  Prints one JSON line.
"""
from __future__ import annotations

import argparse
import json

import torch

from .. import ops
from .roofline import load_peaks


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--heads", type=int, default=20)
    ap.add_argument("--kv-heads", type=int, default=0)
    ap.add_argument("--dim", type=int, default=256)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--skip-baseline", action="store_true")
    args = ap.parse_args()
    assert ops.native_available()
    dev = torch.device("cuda")
    t, H, D = args.tokens, args.heads, args.dim
    Hk = args.kv_heads or H
    q = torch.randn(t, H, D, device=dev).to(torch.bfloat16)
    k = torch.randn(t, Hk, D, device=dev).to(torch.bfloat16)
    v = torch.randn(t, Hk, D, device=dev).to(torch.bfloat16)
    vt = v.permute(1, 2, 0).contiguous()
    out = torch.empty_like(q)
    st = ops.gemm_status(dev)
    flush = torch.empty(160 << 20, dtype=torch.uint8, device=dev)

    def timed(fn):
        for _ in range(min(3, args.iters)):
            fn()
        ts = []
        for _ in range(args.iters):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b) * 1e3)
        return sorted(ts)[len(ts) // 2]

    us = timed(lambda: ops.K.mmb200.fmha_prefill(q, k, vt, out, t, D ** -0.5, st, 0))
    flops = 4.0 * t * t / 2 * H * D
    res = {"bench": "fmha_prefill", "tokens": t, "heads": H, "kv_heads": Hk, "dim": D, "tcgen05_us": round(us, 1),
           "tcgen05_tflops": round(flops / us / 1e6, 1), "status": int(st[0]),
           "frac_of_measured_bf16_peak": round(flops / us / 1e6 / load_peaks()["bf16_tflops"], 3), "timing": "cuda events, median, L2 flushed"}
    if not args.skip_baseline:
        cu = torch.tensor([0, t], dtype=torch.int32, device=dev)
        ops.FMHA_TCGEN05 = False
        us_old = timed(lambda: ops.prefill_attention(q, k, v, cu, cu_k=cu, max_q=t, out=out))
        ops.FMHA_TCGEN05 = True
        res.update(mma_sync_us=round(us_old, 1), mma_sync_tflops=round(flops / us_old / 1e6, 1), speedup=round(us_old / us, 2))
    print(json.dumps(res), flush=True)


if __name__ == "__main__":
    main()
