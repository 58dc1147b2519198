"""Prefill time by op for a (layer-reduced) model preset: every call into the op layer is bracketed by CUDA events.

    python -m metal_marlin_b200.profiling.prefill_bench --model glm-4.7-flash --layers 4 --tokens 4096 --batch 1

Reports milliseconds per op name summed over the prefill, the share of each, and tokens/s extrapolated to the full
layer count.  Parity: the reference's per-component timing tables (``docs/optimization_status_final.md``).
"""
from __future__ import annotations

import argparse
import dataclasses
import json
from collections import defaultdict

import torch

from .. import ops
from ..models.config import get_preset
from ..models.mmfp4_causal_lm import MMFP4ForCausalLM, prefill


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="glm-4.7-flash")
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--iters", type=int, default=3)
    args = ap.parse_args()
    full = get_preset(args.model)
    cfg = dataclasses.replace(full, num_hidden_layers=min(args.layers, full.num_hidden_layers))
    dev = torch.device("cuda")
    lm = MMFP4ForCausalLM.from_config(cfg, device="cuda", seed=0)
    spans = []
    names = ["linear", "bf16_linear", "moe_forward", "moe_router", "rmsnorm", "mla_prep", "rope", "qk_norm_rope_cache", "embedding",
             "bf16_gemm", "silu_mul", "prefill_attention", "fmha_prefill"]
    originals = {n: getattr(ops, n) for n in names}

    def wrap(name, fn):
        def inner(*a, **kw):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            out = fn(*a, **kw)
            e1.record()
            spans.append((name, e0, e1))
            return out
        return inner

    sdpa = torch.nn.functional.scaled_dot_product_attention
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, cfg.vocab_size, (args.tokens,), generator=g).tolist() for _ in range(args.batch)]
    nb = (args.tokens + 16) // 16 + 1
    bt = torch.arange(args.batch * nb, dtype=torch.int32).view(args.batch, nb)
    totals = defaultdict(float)
    wall = []
    for it in range(args.iters + 1):
        kv = lm.new_cache(args.batch * nb, 16)
        spans.clear()
        for n in names:
            setattr(ops, n, wrap(n, originals[n]))
        torch.nn.functional.scaled_dot_product_attention = wrap("sdpa_attention", sdpa)
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        prefill(lm.model, kv, prompts, bt)
        t1.record()
        torch.cuda.synchronize()
        for n in names:
            setattr(ops, n, originals[n])
        torch.nn.functional.scaled_dot_product_attention = sdpa
        if it == 0:
            continue                     # warm-up
        wall.append(t0.elapsed_time(t1))
        for name, e0, e1 in spans:
            totals[name] += e0.elapsed_time(e1) / args.iters
        del kv
    wall_ms = sorted(wall)[len(wall) // 2]
    accounted = sum(totals.values())
    per_layer = (wall_ms - totals.get("bf16_linear", 0.0) - totals.get("embedding", 0.0)) / cfg.num_hidden_layers
    est_full = per_layer * full.num_hidden_layers + totals.get("bf16_linear", 0.0)
    out = {"model": args.model, "layers": cfg.num_hidden_layers, "tokens": args.tokens, "batch": args.batch, "prefill_ms": round(wall_ms, 2),
           "ops_ms": {k: round(v, 2) for k, v in sorted(totals.items(), key=lambda kv: -kv[1])}, "unaccounted_ms": round(wall_ms - accounted, 2),
           "est_full_model_ms": round(est_full, 1), "est_full_model_tok_s": round(args.batch * args.tokens / est_full * 1e3, 0)}
    print(json.dumps(out))


if __name__ == "__main__":
    main()
