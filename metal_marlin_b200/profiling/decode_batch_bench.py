"""Decode step time of one model at several batch sizes and several settings of one dispatch threshold, in one process:

    python -m metal_marlin_b200.profiling.decode_batch_bench --preset glm-4.7-flash --batches 12,16 \\
        --threshold MOE_GEMV_MAX_T --values 16,8 [--prompt-len 512] [--steps 48]

Each combination builds a persistent decode state (CUDA-graph step), prefills random prompts, runs 8 warm-up steps and times
``--steps`` steps with CUDA events; prints one JSON line.  Used to check that a threshold chosen by the kernel-level
auto-tuner also pays off in the whole step.  Parity: reference ``benchmarks/bench_decode_batch.py``-style sweeps.
"""
from __future__ import annotations

import argparse
import json

import torch


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--preset", default="glm-4.7-flash")
    ap.add_argument("--batches", default="12,16")
    ap.add_argument("--threshold", default="MOE_GEMV_MAX_T")
    ap.add_argument("--values", default="16,8")
    ap.add_argument("--prompt-len", type=int, default=512)
    ap.add_argument("--steps", type=int, default=48)
    a = ap.parse_args(argv)
    from .. import ops
    from ..inference.decode import DecodeConfig, DecodeState, persistent_decode_step
    from ..models.mmfp4_causal_lm import MMFP4ForCausalLM
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    lm = MMFP4ForCausalLM.from_config(a.preset, device=dev, seed=0)
    old = getattr(ops, a.threshold)
    res = {}
    try:
        for B in (int(b) for b in a.batches.split(",")):
            for v in (int(x) for x in a.values.split(",")):
                setattr(ops, a.threshold, v)
                st = DecodeState(lm, DecodeConfig(batch_size=B, max_context=a.prompt_len + a.steps + 64, max_new_tokens=a.steps + 16))
                g = torch.Generator().manual_seed(B)
                st.prefill([torch.randint(0, min(1000, lm.config.vocab_size), (a.prompt_len,), generator=g).tolist() for _ in range(B)])
                for _ in range(8):
                    persistent_decode_step(st)
                if dev == "cuda":
                    torch.cuda.synchronize()
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    for _ in range(a.steps):
                        persistent_decode_step(st)
                    e1.record()
                    torch.cuda.synchronize()
                    ms = e0.elapsed_time(e1) / a.steps
                else:
                    import time
                    t0 = time.perf_counter()
                    for _ in range(a.steps):
                        persistent_decode_step(st)
                    ms = (time.perf_counter() - t0) * 1e3 / a.steps
                res[f"batch{B}:{a.threshold}={v}"] = {"ms_per_step": round(ms, 3), "tok_s": round(B * 1e3 / ms, 1)}
                del st
                if dev == "cuda":
                    torch.cuda.empty_cache()
    finally:
        setattr(ops, a.threshold, old)
    print(json.dumps({"bench": "decode_batch", "preset": a.preset, "prompt_len": a.prompt_len, "steps": a.steps, "results": res}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
