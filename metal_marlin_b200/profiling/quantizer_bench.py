"""Quantizer kernels against the PyTorch code they restate, timed on one GPU:

    python -m metal_marlin_b200.profiling.quantizer_bench [--out 4096 --in 4096] [--rtn-shape 16384x8192]

GPTQ of one ``out x in`` layer to FP4 (group 128, block 128) with the block kernel (``ops.gptq_block``) and with the column
loop of PyTorch ops (``ops.force_reference()``), and round-to-nearest E2M1 quantization + packing of a bf16 matrix with the
fused kernel (``ops.fp4_quantize_pack``) and with ``formats.fp4.quantize_codes`` + ``pack_mmfp4``.  Wall clock around a
synchronised call, second run of each; prints one JSON line.  Parity: reference ``benchmarks/bench_quantization.py``.
"""
from __future__ import annotations

import argparse
import json
import time

import torch


def _timed(fn, reps: int = 2) -> float:
    ms = 0.0
    for _ in range(reps):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        fn()
        torch.cuda.synchronize()
        ms = (time.perf_counter() - t0) * 1e3
    return ms


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", type=int, default=4096)
    ap.add_argument("--in", dest="inf", type=int, default=4096)
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--rtn-shape", default="16384x8192")
    a = ap.parse_args(argv)
    from .. import ops
    from ..formats import fp4 as fp4fmt
    from ..quant.gptq import GPTQConfig, gptq_quantize
    torch.manual_seed(0)
    w = torch.randn(a.out, a.inf, device="cuda") * 0.02
    x = torch.randn(a.tokens, a.inf, device="cuda")
    H = x.t() @ x / a.tokens
    cfg = GPTQConfig(fmt="fp4", group_size=128)
    res = {"bench": "quantizer", "gptq_shape": [a.out, a.inf]}
    out = {}
    res["gptq_kernel_ms"] = round(_timed(lambda: out.__setitem__("k", gptq_quantize(w, H, cfg))), 1)

    def loop():
        with ops.force_reference():
            out["t"] = gptq_quantize(w, H, cfg)
    res["gptq_torch_loop_ms"] = round(_timed(loop), 1)
    res["gptq_identical"] = bool(torch.equal(out["k"][0], out["t"][0]) and torch.equal(out["k"][1], out["t"][1]))
    r, c = (int(v) for v in a.rtn_shape.split("x"))
    wb = torch.randn(r, c, device="cuda").to(torch.bfloat16)
    res["rtn_shape"] = [r, c]
    res["rtn_pack_kernel_ms"] = round(_timed(lambda: out.__setitem__("p", ops.fp4_quantize_pack(wb, 128))), 2)
    res["rtn_pack_torch_ms"] = round(_timed(lambda: out.__setitem__("q", fp4fmt.pack_mmfp4(*fp4fmt.quantize_codes(wb, 128)))), 2)
    res["rtn_identical"] = bool(torch.equal(out["p"][0], out["q"][0]) and torch.equal(out["p"][1], out["q"][1]))
    print(json.dumps(res))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
