"""Row-parallel FP4 GEMM with the reduce-scatter epilogue, timed on ONE GPU with the ranks emulated as memory regions
of that GPU (the kernel's "peer" tables point into local buffers), so it can be captured by a single-process profiler.

    python -m metal_marlin_b200.profiling.tp_gemm_bench --tokens 4096 --out 2048 --inner 5120 --tp 2

Reports the GEMM alone, the GEMM with the scatter epilogue (fp32 partial tiles stored to the owner's receive buffer
from the epilogue), the reduce + gather kernel without and with the fused residual add + RMSNorm, the following
column-parallel GEMM with the all-gather wait in its TMA producer (flags pre-set here: the cost of the mechanism, not
of a transfer), and the roofline of the fused step: the slower of FLOPs / measured
bf16 peak and NVLink bytes / 770 GB/s (the bytes a real tp-way run would send).  Multi-GPU numerics of the same
kernels are covered by ``tests/test_tp_fused_gpu.py``.
"""
from __future__ import annotations

import argparse
import json

import torch

from .. import ops
from ..ops.weights import FP4Weight
from .roofline import NVLINK_GBS_PER_DIRECTION, load_peaks


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--out", type=int, default=2048)
    ap.add_argument("--inner", type=int, default=5120, help="full inner dimension; each emulated rank multiplies inner / tp of it")
    ap.add_argument("--tp", type=int, default=2)
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args()
    dev = torch.device("cuda")
    assert ops.native_available()
    M, N, tp = args.tokens, args.out, args.tp
    K = args.inner // tp
    rows = (M + tp - 1) // tp
    W = FP4Weight.from_float(torch.randn(N, K, device=dev) * 0.02, 128)
    x = (torch.randn(M, K, device=dev) * 0.5).to(torch.bfloat16)
    # emulated peers: tp receive buffers and tp gathered buffers, all on this GPU; this process plays rank 0
    rs_bufs = [torch.zeros(tp, rows, N, dtype=torch.float32, device=dev) for _ in range(tp)]
    ag_bufs = [torch.zeros(M, N, dtype=torch.bfloat16, device=dev) for _ in range(tp)]
    rs_flags = [torch.zeros(tp, dtype=torch.int32, device=dev) for _ in range(tp)]
    ag_flags = [torch.zeros(tp, dtype=torch.int32, device=dev) for _ in range(tp)]
    step = torch.ones(1, dtype=torch.int32, device=dev)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    counters = torch.zeros(2, dtype=torch.int32, device=dev)
    tab = lambda ts, off=0: torch.tensor([t.data_ptr() + off for t in ts], dtype=torch.int64).to(dev)
    t_rs_bufs, t_rs_flags, t_ag_bufs, t_ag_flags = tab(rs_bufs), tab(rs_flags), tab(ag_bufs), tab(ag_flags)
    rs_desc = torch.tensor([t_rs_bufs.data_ptr(), t_rs_flags.data_ptr(), counters.data_ptr(), step.data_ptr(), tp, 0, rows], dtype=torch.int64)
    fin_desc = torch.tensor([rs_bufs[0].data_ptr(), rs_flags[0].data_ptr(), t_ag_bufs.data_ptr(), t_ag_flags.data_ptr(), counters[1:].data_ptr(),
                             step.data_ptr(), status.data_ptr(), tp, 0, rows, N, M], dtype=torch.int64)
    # the other emulated ranks never run: mark their partials as delivered
    rs_flags[0].fill_(1 << 30)
    out = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
    st = ops.gemm_status(dev)

    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(args.iters):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) * 1e-3)
        return sorted(ts)[len(ts) // 2]

    t_plain = timed(lambda: ops.K.mmb200.fp4_gemm(x, W.qtile, W.stile, out, N, W.group_size, st))
    t_rs = timed(lambda: ops.K.mmb200.fp4_gemm_rs(x, W.qtile, W.stile, N, W.group_size, st, rs_desc))
    t_fin = timed(lambda: ops.K.mmb200.tp_rs_finish(fin_desc))
    # numerics of the emulation: rank 0's rows of the gathered buffer = sum over slots (only slot 0 is non-zero here)
    ref = (x[:rows].float() @ W.dequantize(torch.float32).t())
    err = float((ag_bufs[0][:rows].float() - ref).abs().max() / ref.abs().max())
    # sequence-parallel boundary: residual add + RMSNorm fused into the reduce kernel, then the next projection gathers
    ag2_bufs = [torch.zeros(M, N, dtype=torch.bfloat16, device=dev) for _ in range(tp)]
    t_ag2 = tab(ag2_bufs)
    resid = (torch.randn(M, N, device=dev) * 0.5).to(torch.bfloat16)
    nw = (1 + 0.1 * torch.randn(N, device=dev)).to(torch.bfloat16)
    t_fin_norm = timed(lambda: ops.K.mmb200.tp_rs_finish_norm(fin_desc, resid, nw, t_ag2.data_ptr(), 1e-6))
    W2 = FP4Weight.from_float(torch.randn(2 * K, N, device=dev) * 0.02, 128)
    out2 = torch.empty(M, 2 * K, dtype=torch.bfloat16, device=dev)
    ag_flags[0].fill_(1 << 30)          # the emulated peers' rows count as delivered
    ag_desc = torch.tensor([ag_flags[0].data_ptr(), step.data_ptr(), tp, 0, rows], dtype=torch.int64)
    t_next = timed(lambda: ops.K.mmb200.fp4_gemm(ag2_bufs[0], W2.qtile, W2.stile, out2, 2 * K, W2.group_size, st))
    t_next_ag = timed(lambda: ops.K.mmb200.fp4_gemm_ag(ag2_bufs[0], W2.qtile, W2.stile, out2, 2 * K, W2.group_size, st, ag_desc))
    part = (x[:rows].float() @ W.dequantize(torch.float32).t()).to(torch.bfloat16).float()
    hn = (part + resid[:rows].float()).to(torch.bfloat16).float()
    xn = (hn * torch.rsqrt(hn.pow(2).mean(-1, keepdim=True) + 1e-6) * nw.float())
    err_norm = float((ag2_bufs[0][:rows].float() - xn).abs().max() / xn.abs().max())
    ref2 = ag2_bufs[0][:rows].float() @ W2.dequantize(torch.float32).t()
    err_ag = float((out2[:rows].float() - ref2).abs().max() / ref2.abs().max())
    flops = 2.0 * M * N * K
    peaks = load_peaks()
    nv_bytes = (tp - 1) / tp * M * N * 4 + (tp - 1) / tp * M * N * 2      # scatter fp32 partials out + gather bf16 rows out, per rank
    roof = max(flops / (peaks["bf16_tflops"] * 1e12), nv_bytes / (NVLINK_GBS_PER_DIRECTION * 1e9))
    print(json.dumps({"M": M, "N": N, "K_per_rank": K, "tp": tp, "gemm_us": round(t_plain * 1e6, 1), "gemm_rs_us": round(t_rs * 1e6, 1),
                      "rs_finish_us": round(t_fin * 1e6, 1), "rs_finish_norm_us": round(t_fin_norm * 1e6, 1),
                      "next_gemm_us": round(t_next * 1e6, 1), "next_gemm_ag_wait_us": round(t_next_ag * 1e6, 1),
                      "rel_err_norm": round(err_norm, 5), "rel_err_ag_gemm": round(err_ag, 5), "gemm_tflops": round(flops / t_plain / 1e12, 1),
                      "gemm_rs_tflops": round(flops / t_rs / 1e12, 1), "nvlink_bytes_per_rank": int(nv_bytes), "roof_us": round(roof * 1e6, 1),
                      "fraction_of_roof": round(roof / (t_rs + t_fin), 3), "of": peaks["source"], "rel_err": round(err, 5), "status": int(status[0])}))


if __name__ == "__main__":
    main()
