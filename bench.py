#!/usr/bin/env python
"""Headline benchmark: GLM-4.7-Flash-architecture MMFP4 decode throughput on B200.

    python bench.py --gpus N --steps K --warmup W [--batch B] [--prompt-len P] [--impl ours|reference|eager]

Workload (the reference's headline, ``README.md:23-24`` of RESMP-DEV/metal-marlin: GLM-4.7-Flash
MMFP4 decode, 35.2 tok/s at batch 1): random-init weights of the GLM-4.7-Flash architecture
RTN-quantized to MMFP4 (group 128), paged latent KV cache with 16-token blocks, a uniform-random
prompt of ``--prompt-len`` tokens (default 4096) prefilled through the engine, then greedy decode.
A step = one decode iteration of the whole batch (all layers, head, sampler).

Timing: W untimed warm-up steps, then exactly K steps between CUDA events on the launching stream
with a barrier + synchronize on both sides, max over ranks.  Each step streams ~2.3 GB of weights,
far more than the 126 MB L2, so no explicit flush is needed (stated in ``config``).
The ``e2e`` number drives the same steps through the public session API with, per step, a
host->device copy of the step's input ids from pinned memory and a device->host read of the sampled ids.

One JSON line is printed by rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

BASELINE_TOK_S = 35.2   # reference headline (Apple M4 Max), README.md:23


def _args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=1, help="sequences per model replica")
    ap.add_argument("--prompt-len", type=int, default=4096)
    ap.add_argument("--model", default="glm-4.7-flash")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "eager"])
    ap.add_argument("--parallelism", default="auto", choices=["auto", "tp", "dp"])
    ap.add_argument("--extra", action="store_true", help="also measure batch 32 and prefill (TTFT)")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--kv-dtype", default="bf16", choices=["bf16", "fp8"], help="paged KV cache element type (fp8: E4M3 + per-row scale)")
    ap.add_argument("--no-graph", action="store_true", help="launch the decode step kernel by kernel (profiling)")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.gpu)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, reasons, power = [], [], set(), []
        for r in self.rows:
            f = [x.strip() for x in r.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
                power.append(float(f[3]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


def reference_arm(args):
    """Drive the unmodified reference package (installed under baseline/_ref) through its stock loader.

    A random-init checkpoint of the GLM-4.7-Flash architecture family is written in the shared MMFP4 format and handed to
    the reference's ``metal_marlin.model_utils.load_prequantized_mmfp4_model(path, device="cuda")``.  On a machine without
    Apple's MPS backend that loader cannot build its quantized layers (``MetalQuantizedLinear.__init__`` calls
    ``require_mps()``; ``replace_linear_layers`` swallows the error and leaves ``nn.Linear`` modules, so the packed tensors
    then fail to copy), and ``MMFP4Pipeline.from_pretrained`` imports ``metal_marlin.models.mmfp4_causal_lm``, which the
    reference tree does not contain.  The exact exception text is reported in the ``unavailable`` line.  If the loader ever
    succeeds, the same decode steps are timed through the reference model's own forward."""
    import tempfile
    root = os.path.dirname(os.path.abspath(__file__))
    ref_dir = os.path.join(root, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "metal_marlin")):
        print(json.dumps({"impl": "reference", "unavailable":
                          "baseline/_ref is not installed (pip install --no-deps --target baseline/_ref <reference checkout>)"}))
        return 0
    why = []
    model = None
    with tempfile.TemporaryDirectory() as tmp:
        try:
            # checkpoint writer only (file format shared with the reference); nothing of this repo runs after this block
            from metal_marlin_b200.models.config import get_preset
            from metal_marlin_b200.quant.convert import save_random_checkpoint
            preset = os.environ.get("MMB200_REF_PRESET", "tiny-mla-moe")
            save_random_checkpoint(get_preset(preset), tmp, fmt="mmfp4", seed=args.seed)
            for m in [m for m in sys.modules if m.startswith("metal_marlin_b200")]:
                del sys.modules[m]
        except Exception as e:
            print(json.dumps({"impl": "reference", "unavailable": f"could not write the synthetic checkpoint: {e!r}"[:300]}))
            return 0
        sys.path.insert(0, ref_dir)
        import io
        import contextlib
        import torch
        dev = "cuda" if torch.cuda.is_available() else "cpu"
        try:
            with contextlib.redirect_stdout(io.StringIO()):
                from metal_marlin.inference_metal import MetalQuantizedLinear
                MetalQuantizedLinear(in_features=256, out_features=256, bits=4, group_size=64, bias=False)
        except Exception as e:
            why.append(f"MetalQuantizedLinear: {type(e).__name__}: {' '.join(str(e).split())[:120]}")
        try:
            with contextlib.redirect_stdout(io.StringIO()):
                from metal_marlin.model_utils import load_prequantized_mmfp4_model
                model, _tok = load_prequantized_mmfp4_model(tmp, device=dev)
        except Exception as e:
            why.append(f"load_prequantized_mmfp4_model(device={dev!r}): {type(e).__name__}: {' '.join(str(e).split())[:160]}")
        try:
            with contextlib.redirect_stdout(io.StringIO()):
                from metal_marlin.inference.mmfp4_pipeline import MMFP4Pipeline as RefPipeline
                RefPipeline.from_pretrained(tmp)
        except Exception as e:
            why.append(f"MMFP4Pipeline.from_pretrained: {type(e).__name__}: {' '.join(str(e).split())[:120]}")
    if model is None or why:
        print(json.dumps({"impl": "reference", "unavailable": "reference is Apple-Metal only; stock CUDA path fails: " + " | ".join(why)}))
        return 0
    # the loader worked: time its own forward, one token per step, batch 1
    model = model.to(dev).eval()
    ids = torch.randint(0, model.config.vocab_size, (1, args.prompt_len), device=dev)
    with torch.no_grad():
        out = model(ids, use_cache=True)
        past, tok = out.past_key_values, out.logits[:, -1:].argmax(-1)
        for _ in range(max(args.warmup, 3)):
            out = model(tok, past_key_values=past, use_cache=True)
            past, tok = out.past_key_values, out.logits[:, -1:].argmax(-1)
        t0 = time.perf_counter()
        if dev == "cuda":
            torch.cuda.synchronize()
        for _ in range(args.steps):
            out = model(tok, past_key_values=past, use_cache=True)
            past, tok = out.past_key_values, out.logits[:, -1:].argmax(-1)
        if dev == "cuda":
            torch.cuda.synchronize()
        ms = (time.perf_counter() - t0) * 1e3 / args.steps
    print(json.dumps({"impl": "reference", "metric": "glm47_flash_mmfp4_decode_tok_s_bs1", "value": 1e3 / ms, "unit": "tok/s",
                      "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
                      "config": {"model": os.environ.get("MMB200_REF_PRESET", "tiny-mla-moe"), "note": "reference loader succeeded"}}))
    return 0


def main():
    args = _args()
    if args.impl == "reference":
        # the reference is a single-device program: under a multi-rank launch only rank 0 runs it and prints the line
        if int(os.environ.get("RANK", "0")) != 0:
            return 0
        return reference_arm(args)

    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        # a rank that fails alone (an exception the others do not see) must not leave the others waiting in a collective for
        # the library's ten-minute default: collectives give up after three minutes and the error is reported in the line
        import datetime
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=180))

    from metal_marlin_b200 import ops
    from metal_marlin_b200.engine.session import DecodeSession, SamplingParams
    from metal_marlin_b200.models.config import get_preset
    from metal_marlin_b200.models.mmfp4_causal_lm import MMFP4ForCausalLM, prefill

    cfg = get_preset(args.model)
    block_size = 16

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    eager = args.impl == "eager"
    t_build = time.time()
    lm = MMFP4ForCausalLM.from_config(cfg, device=str(dev), seed=args.seed)
    # N > 1: the headline is data parallel (one replica per GPU, each decoding its own stream: weak scaling);
    # the same run then times the tensor-parallel latency mode (one model over all GPUs, partial sums exchanged
    # inside the kernels over NVLink) and reports it under "tp".  --parallelism tp makes that the headline.
    headline_tp = world > 1 and args.parallelism == "tp"
    also_tp = world > 1 and args.parallelism == "auto" and not (args.impl == "eager")
    state = {"model": lm.model, "tp": False, "ctx": None}

    def to_tensor_parallel():
        # every rank built the same weights (per-tensor seeds); keep only this rank's tensor-parallel shard
        from metal_marlin_b200.parallel.tp import make_context, shard_transformer
        state["ctx"] = make_context(cfg, dev, mode="fused")
        state["model"] = shard_transformer(lm.model, rank, world, state["ctx"])
        state["tp"] = True

    if headline_tp:
        to_tensor_parallel()
    build_s = time.time() - t_build
    if eager:
        from metal_marlin_b200.baseline_eager import EagerBF16Model
        eager_model = EagerBF16Model(lm.model)

    def run_config(batch: int, steps: int, warmup: int, e2e: bool, graph: bool = True, same_batch=None):
        total_len = args.prompt_len + warmup + steps * (2 if e2e else 1) + 8
        nb = (total_len + block_size - 1) // block_size
        kv = lm.new_cache(batch * nb, block_size, kv_dtype=args.kv_dtype)
        use_tp, run_model = state["tp"], state["model"]
        if same_batch is None:
            same_batch = use_tp
        g = torch.Generator().manual_seed(args.seed + (0 if same_batch else rank))     # tensor-parallel ranks share the batch
        prompts = [torch.randint(0, cfg.vocab_size, (args.prompt_len,), generator=g).tolist() for _ in range(batch)]
        bt = torch.arange(batch * nb, dtype=torch.int32).view(batch, nb)
        # one untimed prefill of the first sequence: one-time library / attribute initialisation is not time-to-first-token
        # (the timed prefill below rewrites the same cache blocks)
        if eager:
            eager_model.prefill(kv, prompts[:1], bt[:1])
        else:
            prefill(run_model, kv, prompts[:1], bt[:1])
        torch.cuda.synchronize(dev)
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        if eager:
            logits = eager_model.prefill(kv, prompts, bt)
        else:
            logits = prefill(run_model, kv, prompts, bt)
        ev1.record()
        torch.cuda.synchronize(dev)
        ttft_ms = ev0.elapsed_time(ev1)
        model = eager_model if eager else run_model
        no_graph = eager or args.no_graph or not graph
        sess = DecodeSession(model, kv, batch, nb, max_new_tokens=0, max_ctx=total_len, use_graph=not no_graph)
        sess.set_sampling([SamplingParams()] * batch)
        first = run_model.greedy(logits) if not eager else logits.argmax(-1)
        sess.set_state(first, [args.prompt_len] * batch, bt)
        l0 = ops.launch_count()
        sess._step_body() if no_graph else sess.capture()
        launches_per_step = (ops.launch_count() - l0) // (1 if no_graph else 3)
        if no_graph:
            sess.set_state(first, [args.prompt_len] * batch, bt)
        for _ in range(warmup):
            sess.step()
        barrier()
        sampler = ClockSampler(local_rank)
        sampler.start()
        time.sleep(0.3)
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        s0.record()
        for _ in range(steps):
            sess.step()
        s1.record()
        barrier()
        ms = max_over_ranks(s0.elapsed_time(s1))
        clocks = sampler.stop()
        res = {"ms_per_step": ms / steps, "ttft_ms": max_over_ranks(ttft_ms), "launches_per_step": launches_per_step,
               "clocks": clocks}
        if e2e:
            # public-API loop: pinned-host ids in, sampled ids out, every step
            h_in = torch.empty(batch, dtype=torch.int64).pin_memory()
            h_out = torch.empty(batch, dtype=torch.int64).pin_memory()
            h_in.copy_(sess.out_ids.cpu())
            barrier()
            t0 = time.perf_counter()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                sess.ids.copy_(h_in, non_blocking=True)          # H2D: this step's input token ids
                sess.step()
                h_out.copy_(sess.out_ids, non_blocking=True)     # D2H: the step's result
                torch.cuda.current_stream(dev).synchronize()
                h_in.copy_(h_out)
            e1.record()
            barrier()
            wall_ms = (time.perf_counter() - t0) * 1e3
            res["e2e_ms_per_step"] = max_over_ranks(max(wall_ms, e0.elapsed_time(e1))) / steps
            res["h2d_bytes_per_step"] = batch * 8
            res["d2h_bytes_per_step"] = batch * 8
        del sess, kv
        torch.cuda.empty_cache()
        return res

    use_tp = state["tp"]
    replicas = 1 if use_tp else world
    r = run_config(args.batch, args.steps, args.warmup, e2e=True)
    tok_s = replicas * args.batch * 1e3 / r["ms_per_step"]
    e2e_tok_s = replicas * args.batch * 1e3 / r["e2e_ms_per_step"]
    out = {
        "metric": f"{args.model.replace('-', '_').replace('.', '')}_mmfp4_decode_tok_s_bs{args.batch}".replace("glm_47_flash", "glm47_flash"),
        "value": round(tok_s, 2), "unit": "tok/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(r["ms_per_step"], 4), "higher_is_better": True, "scaling": "strong" if use_tp else "weak",
        "vs_baseline": round(tok_s / BASELINE_TOK_S, 2), "dtype": "bf16", "data": "synthetic",
        "impl": args.impl,
        "config": {"model": f"{args.model} (random-init, RTN MMFP4 group 128)", "global_batch": replicas * args.batch,
                   "seq_len": args.prompt_len,
                   "parallelism": (f"tp{world} (in-kernel NVLink exchange)" if use_tp else f"dp{world}") if world > 1 else "single",
                   "kv": f"paged, 16-token blocks, {args.kv_dtype}", "decode": "greedy, CUDA graph per step",
                   "l2_policy": "inputs larger than L2 (each step streams >2 GB of weights)",
                   "weights_gb_per_gpu": round(state["model"].weight_bytes() / 1e9, 2), "build_s": round(build_s, 1)},
        "clocks": r["clocks"],
        "e2e": {"value": round(e2e_tok_s, 2), "unit": "tok/s", "h2d_bytes_per_step": r["h2d_bytes_per_step"],
                "d2h_bytes_per_step": r["d2h_bytes_per_step"], "ms_per_step": round(r["e2e_ms_per_step"], 4)},
        "gpu_launches": int(r["launches_per_step"] * args.steps),
        "ttft_ms_p50": round(r["ttft_ms"], 2),
    }
    if use_tp:
        out["config"]["exchange_status"] = state["ctx"].check()
    n_half, w_half = max(8, args.steps // 2), max(3, args.warmup // 2)
    if args.extra or world > 1 or args.batch == 1:
        # batch 32 per replica (decode throughput regime) and its time to first token
        try:
            r32 = run_config(32, n_half, w_half, e2e=False)
            out["extra"] = {"bs32_tok_s": round((1 if state["tp"] else world) * 32 * 1e3 / r32["ms_per_step"], 1),
                            "bs32_ms_per_step": round(r32["ms_per_step"], 4), "bs32_ttft_ms": round(r32["ttft_ms"], 1),
                            "bs32_launches_per_step": r32["launches_per_step"]}
        except Exception as e:      # the headline line must still be printed
            out["extra"] = {"error": repr(e)[:300]}
    failed_section = False
    if world > 1 and args.parallelism == "auto" and not eager and cfg.is_moe:
        # expert parallel with data-parallel attention: every rank serves its own sequences, the MoE layers exchange token
        # rows with the expert owners - inside this library's kernels over NVLink ("fused"), or through NCCL all-to-all
        try:
            from metal_marlin_b200.parallel.ep import shard_transformer_ep
            ep_out = {"parallelism": f"ep{world} (attention data parallel, experts sharded)", "global_batch": 32 * world,
                      "prompt_tokens_per_rank": 32 * args.prompt_len}
            saved = dict(state)
            for arm in ("fused", "nccl"):
                state["model"] = shard_transformer_ep(lm.model, rank, world, 8192, mode=arm)
                state["model"].ep.uniform = True      # every rank brings the same number of tokens to every pass
                state["tp"] = False
                re = run_config(32, n_half, w_half, e2e=False, graph=(arm == "fused"), same_batch=False)
                ep_out[arm] = {"bs32_per_rank_tok_s": round(world * 32 * 1e3 / re["ms_per_step"], 1),
                               "ms_per_step": round(re["ms_per_step"], 4),
                               "prefill_tok_s": round(world * 32 * args.prompt_len * 1e3 / re["ttft_ms"], 1),
                               "prefill_ms": round(re["ttft_ms"], 1), "launches_per_step": re["launches_per_step"],
                               "exchange_status": state["model"].ep.check()}
                state["model"] = None
                torch.cuda.empty_cache()
            state.update(saved)
            out["ep"] = ep_out
        except Exception as e:
            out["ep"] = {"error": repr(e)[:300]}
            failed_section = True
    if also_tp and not failed_section:
        # latency mode on the same GPUs: one stream, every matrix split over the ranks
        try:
            to_tensor_parallel()
            rt = run_config(args.batch, args.steps, args.warmup, e2e=False)
            out["tp"] = {"parallelism": f"tp{world} (in-kernel NVLink exchange)", "global_batch": args.batch,
                         "ms_per_step": round(rt["ms_per_step"], 4), "tok_s": round(args.batch * 1e3 / rt["ms_per_step"], 2),
                         "ttft_ms": round(rt["ttft_ms"], 2),      # prompt split over the ranks: GEMM -> reduce-scatter -> gather -> GEMM in-kernel
                         "launches_per_step": rt["launches_per_step"], "multimem": bool(getattr(state["ctx"], "use_multimem", False)),
                         "symmetric_memory": getattr(getattr(state["ctx"], "buf", None), "backend", None),
                         "weights_gb_per_gpu": round(state["model"].weight_bytes() / 1e9, 2)}
            rt32 = run_config(32, n_half, w_half, e2e=False)
            out["tp"].update(bs32_tok_s=round(32 * 1e3 / rt32["ms_per_step"], 1), bs32_ms_per_step=round(rt32["ms_per_step"], 4),
                             bs32_ttft_ms=round(rt32["ttft_ms"], 1), exchange_status=state["ctx"].check())
        except Exception as e:
            out["tp"] = dict(out.get("tp") or {}, error=repr(e)[:300])
            failed_section = True
    if rank == 0:
        print(json.dumps(out), flush=True)
    if world > 1:
        if failed_section:
            # the ranks may have left the tensor-parallel section at different points: no further collective, no group teardown
            sys.stdout.flush()
            os._exit(0)
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
