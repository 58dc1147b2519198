"""Qwen3-30B-A3B-architecture MoE quantized to trellis-v2 (mixed 2-4 bits per expert), expert parallel over the GPUs of the job.

    python bench/trellis_ep.py --seqs 256 --prompt-len 2048                                   # one GPU, no exchange
    torchrun --nproc-per-node 8 --master-addr 127.0.0.1 bench/trellis_ep.py --seqs 256 --prompt-len 2048

Random-init weights drawn in the quantized domain (``TrellisRandomSource``), uniform-random token ids.  Attention and the dense
layers are replicated (every rank serves ``seqs / N`` sequences); the routed experts are split over the ranks and the MoE
layers exchange token rows inside this library's kernels over NVLink peer memory ("fused"), or through NCCL all-to-all
("nccl", the baseline).  Expert matrices are decoded from their 2-4 bit code streams inside the tensor-core GEMM's main
loop.  Prints one JSON line: prompt tokens per second (prefill of ``seqs`` x ``prompt-len``) and decode tokens per second at
batch ``seqs`` (whole job), timed on the device, max over ranks.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen3-30b-a3b")
    ap.add_argument("--seqs", type=int, default=256, help="sequences of the whole job")
    ap.add_argument("--prompt-len", type=int, default=2048)
    ap.add_argument("--steps", type=int, default=16)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--layers", type=int, default=0, help="truncate the model (0 = all layers)")
    ap.add_argument("--arms", default="fused,nccl")
    ap.add_argument("--seed", type=int, default=0)
    args = ap.parse_args()
    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import datetime
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=180))
    from metal_marlin_b200 import ops
    from metal_marlin_b200.engine.session import DecodeSession, SamplingParams
    from metal_marlin_b200.models.config import get_preset
    from metal_marlin_b200.models.mmfp4_causal_lm import prefill
    from metal_marlin_b200.parallel.ep import shard_transformer_ep
    from metal_marlin_b200.trellis.lm import TrellisForCausalLM

    cfg = get_preset(args.model)
    if args.layers:
        cfg.num_hidden_layers = args.layers
    t0 = time.time()
    lm = TrellisForCausalLM.from_config(cfg, device=str(dev), seed=args.seed, expert_bits=(2, 3, 4))
    build_s = time.time() - t0
    B = max(1, args.seqs // world)
    bs = 16
    total = args.prompt_len + args.warmup + args.steps + 8
    nb = (total + bs - 1) // bs

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def mx(v):
        if world == 1:
            return v
        t = torch.tensor([v], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def run(model, graph):
        kv = lm.new_cache(B * nb, bs)
        g = torch.Generator().manual_seed(args.seed + rank)
        prompts = [torch.randint(0, cfg.vocab_size, (args.prompt_len,), generator=g).tolist() for _ in range(B)]
        bt = torch.arange(B * nb, dtype=torch.int32).view(B, nb)
        prefill(model, kv, prompts[:1], bt[:1])            # untimed: one-time initialisation
        sync()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        logits = prefill(model, kv, prompts, bt)
        e1.record()
        torch.cuda.synchronize(dev)
        prefill_ms = mx(e0.elapsed_time(e1))
        sess = DecodeSession(model, kv, B, nb, max_new_tokens=0, max_ctx=total, use_graph=graph)
        sess.set_sampling([SamplingParams()] * B)
        sess.set_state(logits.argmax(-1), [args.prompt_len] * B, bt)
        for _ in range(args.warmup):
            sess.step()
        sync()
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record()
        for _ in range(args.steps):
            sess.step()
        s1.record()
        sync()
        ms = mx(s0.elapsed_time(s1)) / args.steps
        del sess, kv
        torch.cuda.empty_cache()
        return {"prefill_tok_s": round(world * B * args.prompt_len * 1e3 / prefill_ms, 1), "prefill_ms": round(prefill_ms, 1),
                "decode_tok_s": round(world * B * 1e3 / ms, 1), "decode_ms_per_step": round(ms, 3)}

    out = {"metric": "qwen3_30b_a3b_trellis_v2_expert_parallel", "n_gpus": world, "seqs": world * B, "prompt_len": args.prompt_len,
           "steps": args.steps, "warmup": args.warmup, "dtype": "bf16 activations, 2-4 bit trellis experts, 4-bit trellis dense matrices",
           "data": "synthetic", "layers": cfg.num_hidden_layers, "build_s": round(build_s, 1)}
    try:
        if world == 1:
            out["single"] = run(lm.model, graph=True)
        else:
            for arm in [a for a in args.arms.split(",") if a]:
                model = shard_transformer_ep(lm.model, rank, world, 8192, mode=arm)
                model.ep.uniform = True
                out[arm] = run(model, graph=(arm == "fused"))
                out[arm]["exchange_status"] = model.ep.check()
                del model
                torch.cuda.empty_cache()
        out["status"] = ops.check_status(dev)
    except Exception as e:
        out["error"] = repr(e)[:400]
    if rank == 0:
        print(json.dumps(out), flush=True)
    if world > 1:
        if "error" in out:
            os._exit(0)
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
