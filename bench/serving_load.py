"""Serving load test: Poisson arrivals into the continuous-batching engine, synthetic prompts.

    python bench/serving_load.py --model glm-4.7-flash --rate 16 --requests 64 --prompt-min 128 --prompt-max 1024 \
        --out-min 32 --out-max 128 [--speculative ngram | draft --draft-layers 2 --num-spec 4]
    torchrun --nproc-per-node 8 --master-addr 127.0.0.1 bench/serving_load.py --model qwen3.5-122b-a10b --tp 8 --ep 8 \
        --speculative draft --rate 16 --prompt-max 4096 --out-min 64 --out-max 512

Requests are submitted from a driver thread at exponentially distributed intervals while the engine loop (paged KV,
chunked prefill, CUDA-graph decode buckets, optional speculative decoding in the pipeline layer) runs in its own
thread - the in-process equivalent of the OpenAI server's request path without HTTP parsing.  Prints one JSON line:
p50 / p99 time-to-first-token, p50 / p99 end-to-end latency, output tokens per second over the busy interval.

Parity: the reference's acceptance thresholds for its server (``docs/VALIDATION_CHECKLIST.md:66,78``: >= 100 tok/s
aggregate at 5 concurrent requests) and ``tests/validation/test_e2e_validation.py``.
"""
from __future__ import annotations

import argparse
import json
import os
import random
import sys
import threading
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

from metal_marlin_b200.engine.engine import EngineConfig, LLMEngine  # noqa: E402
from metal_marlin_b200.engine.request import GenerationRequest  # noqa: E402
from metal_marlin_b200.engine.session import SamplingParams  # noqa: E402
from metal_marlin_b200.models.mmfp4_causal_lm import MMFP4ForCausalLM  # noqa: E402


def pct(xs, q):
    xs = sorted(xs)
    if not xs:
        return None
    return xs[min(len(xs) - 1, int(q * len(xs)))]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="glm-4.7-flash")
    ap.add_argument("--rate", type=float, default=16.0, help="mean arrivals per second")
    ap.add_argument("--requests", type=int, default=64)
    ap.add_argument("--prompt-min", type=int, default=128)
    ap.add_argument("--prompt-max", type=int, default=1024)
    ap.add_argument("--out-min", type=int, default=32)
    ap.add_argument("--out-max", type=int, default=128)
    ap.add_argument("--max-seqs", type=int, default=32)
    ap.add_argument("--kv-blocks", type=int, default=8192)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--device", default=None)
    ap.add_argument("--tp", type=int, default=1, help="tensor-parallel degree (under torchrun)")
    ap.add_argument("--ep", type=int, default=1, help="expert-parallel degree (with --tp: whole experts per rank)")
    ap.add_argument("--speculative", default="none", choices=["none", "ngram", "draft"],
                    help="draft: a random-init small model of the same vocabulary (--draft-layers)")
    ap.add_argument("--draft-layers", type=int, default=2)
    ap.add_argument("--num-spec", type=int, default=4)
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    ecfg = EngineConfig(num_kv_blocks=args.kv_blocks, block_size=16, max_model_len=args.prompt_max + args.out_max + 16,
                        max_num_seqs=args.max_seqs, max_num_batched_tokens=4096, max_prefill_tokens=2048, max_chunk=1024,
                        use_cuda_graphs=torch.cuda.is_available(), request_timeout_s=600.0)
    if world > 1:
        from metal_marlin_b200.engine.distributed import ParallelConfig, build_engine, init_process_group
        rank, world, device, ctrl = init_process_group()
        dev = str(device)
        lm = MMFP4ForCausalLM.from_config(args.model, device=dev, seed=args.seed)
        pc = ParallelConfig.parse(tp=args.tp, ep=args.ep, world=world)
        eng = build_engine(lm.model, ecfg, pc, rank, world, device, ctrl)
        core = eng.engine
    else:
        rank = 0
        dev = args.device or ("cuda" if torch.cuda.is_available() else "cpu")
        lm = MMFP4ForCausalLM.from_config(args.model, device=dev, seed=args.seed)
        eng = core = LLMEngine(lm.model, ecfg)
        pc = None
    cfg = lm.config
    if args.speculative != "none" and rank == 0:
        draft = "ngram"
        if args.speculative == "draft":        # small random-init model with the target's vocabulary
            import copy
            dcfg = copy.copy(cfg)
            dcfg.num_hidden_layers = args.draft_layers
            dcfg.first_k_dense_replace = min(dcfg.first_k_dense_replace, args.draft_layers)
            draft = MMFP4ForCausalLM.from_config(dcfg, device=dev, seed=args.seed + 1)
        core.enable_speculative(draft, num_speculative_tokens=args.num_spec)
    if rank != 0:
        eng.serve_forever()
        return
    rng = random.Random(args.seed)
    g = torch.Generator().manual_seed(args.seed)
    # warm-up: compile the graph buckets and the prefill shapes
    eng.generate([torch.randint(0, cfg.vocab_size, (args.prompt_min,), generator=g).tolist()] * 2, max_new_tokens=4)
    eng.start()
    rrs = []
    t_start = time.monotonic()

    def driver():
        for _ in range(args.requests):
            time.sleep(rng.expovariate(args.rate))
            n_in = rng.randint(args.prompt_min, args.prompt_max)
            n_out = rng.randint(args.out_min, args.out_max)
            ids = torch.randint(0, cfg.vocab_size, (n_in,), generator=g).tolist()
            rrs.append(eng.add_request(GenerationRequest(ids, n_out, SamplingParams(), timeout_s=600.0)))

    th = threading.Thread(target=driver)
    th.start()
    th.join()
    for rr in rrs:
        rr.done.wait(timeout=600)
    t_end = time.monotonic()
    eng.stop()
    done = [rr for rr in rrs if rr.finish_time is not None]
    ttft = [rr.first_token_time - rr.arrival for rr in done if rr.first_token_time is not None]
    e2e = [rr.finish_time - rr.arrival for rr in done]
    out_tokens = sum(len(rr.output_ids) for rr in done)
    print(json.dumps({
        "model": args.model, "rate_req_s": args.rate, "requests": args.requests, "completed": len(done),
        "prompt_len": [args.prompt_min, args.prompt_max], "output_len": [args.out_min, args.out_max],
        "ttft_ms_p50": round(1e3 * pct(ttft, 0.5), 1) if ttft else None, "ttft_ms_p99": round(1e3 * pct(ttft, 0.99), 1) if ttft else None,
        "latency_ms_p50": round(1e3 * pct(e2e, 0.5), 1) if e2e else None, "latency_ms_p99": round(1e3 * pct(e2e, 0.99), 1) if e2e else None,
        "output_tok_s": round(out_tokens / max(t_end - t_start, 1e-9), 1), "engine_iterations": eng.iterations, "wall_s": round(t_end - t_start, 2),
        "parallelism": pc.mode if pc is not None else "single", "n_gpus": world, "speculative": args.speculative,
        "spec_acceptance_rate": round(core.spec_accepted / max(1, core.spec_proposed), 3) if core.spec is not None else None,
        "exchange_status": eng.check() if hasattr(eng, "check") else 0}))


if __name__ == "__main__":
    main()
