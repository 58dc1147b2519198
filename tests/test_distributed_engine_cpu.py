"""The multi-GPU serving engines on CPU ranks (gloo, real processes): tensor parallel (leader announces every batch, the
other shard replays it), tensor + expert parallel (whole experts per rank) and expert parallel with data-parallel
attention (lockstep engines, requests dealt out by rank 0, filler passes on idle ranks) must return exactly the tokens
the single-process engine returns.  Reference behaviour: sharded-vs-unsharded equality of
metal_marlin/distributed/verification.py:85-509."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


PROMPTS = [list(range(3, 40)), list(range(50, 58)), [7, 7, 7, 9], list(range(100, 170)), [1, 2, 3, 4, 5]]


def _expected(preset, seed, new_tokens, parts=1):
    """Single-process result.  ``parts``: the requests are dealt round-robin to that many engines, as the expert-parallel
    group deals them to its ranks, so every sequence meets the same batch mates (CPU matrix products round differently for
    different batch sizes, and a random-init model has near-ties)."""
    from metal_marlin_b200.engine.engine import EngineConfig, LLMEngine
    from metal_marlin_b200.models.mmfp4_causal_lm import MMFP4ForCausalLM
    lm = MMFP4ForCausalLM.from_config(preset, device="cpu", seed=seed)
    _sharpen(lm.model)
    out = [None] * len(PROMPTS)
    for r in range(parts):
        eng = LLMEngine(lm.model, EngineConfig(num_kv_blocks=64, block_size=16, max_model_len=128, max_chunk=128,
                                               max_prefill_tokens=512, use_cuda_graphs=False))
        idx = list(range(r, len(PROMPTS), parts))
        for i, o in zip(idx, eng.generate([PROMPTS[i] for i in idx], max_new_tokens=new_tokens)):
            out[i] = o
    return out


def _sharpen(model):
    """Larger router logits: the top-k choice must not hinge on the last bit of a sum whose order differs between layouts."""
    for L in model.layers:
        if L.router_w is not None:
            L.router_w.mul_(16.0)


def _worker(rank, world, port, mode, preset, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    try:
        from metal_marlin_b200.engine.distributed import ParallelConfig, build_engine, init_process_group
        from metal_marlin_b200.engine.engine import EngineConfig
        from metal_marlin_b200.models.mmfp4_causal_lm import MMFP4ForCausalLM
        r, w, dev, ctrl = init_process_group(torch.device("cpu"))
        lm = MMFP4ForCausalLM.from_config(preset, device="cpu", seed=5)
        _sharpen(lm.model)
        pc = {"tp": ParallelConfig.parse(tp=world, world=world), "tp+ep": ParallelConfig.parse(tp=world, ep=world, world=world),
              "ep": ParallelConfig.parse(ep=world, world=world, exchange="nccl")}[mode]
        assert pc.mode == mode
        cfg = EngineConfig(num_kv_blocks=64, block_size=16, max_model_len=128, max_chunk=128, max_prefill_tokens=512,
                           use_cuda_graphs=False)
        de = build_engine(lm.model, cfg, pc, r, w, dev, ctrl)
        if de.is_leader:
            out = de.generate(PROMPTS, max_new_tokens=5)
            extra = de.generate(PROMPTS[:1], max_new_tokens=3)          # a second wave on a running group
            de.stop()
            q.put((rank, {"out": out, "extra": extra, "status": de.check()}))
        else:
            de.serve_forever()
            q.put((rank, {"iterations": de.engine.iterations, "status": de.check()}))
    except Exception as e:          # surface the failure instead of a silent time-out
        import traceback
        q.put((rank, {"error": traceback.format_exc()}))
        raise
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


@pytest.mark.parametrize("mode,preset", [("tp", "tiny-llama"), ("tp", "tiny-mla-moe"), ("tp+ep", "tiny-mla-moe"), ("ep", "tiny-mla-moe")])
def test_multi_rank_engine_matches_single_process(mode, preset):
    world = 2
    want = _expected(preset, 5, 5, parts=world if mode == "ep" else 1)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, mode, preset, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=600) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
    for r in range(world):
        assert "error" not in results[r], results[r]["error"]
        assert results[r]["status"] == 0
    assert results[0]["out"] == want, (results[0]["out"], want)
    assert results[0]["extra"][0] == want[0][:3]
    if mode == "ep":
        assert results[1]["iterations"] > 0          # the other rank served requests of its own


def test_parallel_config_validation():
    from metal_marlin_b200.engine.distributed import ParallelConfig
    assert ParallelConfig.parse(world=1).mode == "single"
    assert ParallelConfig.parse(tp=4, world=4).mode == "tp"
    assert ParallelConfig.parse(tp=2, dp=2, world=4).mode == "tp"
    assert ParallelConfig.parse(ep=8, world=8).mode == "ep"
    assert ParallelConfig.parse(tp=8, ep=8, world=8).mode == "tp+ep"
    with pytest.raises(ValueError):
        ParallelConfig.parse(tp=4, world=8)
    with pytest.raises(ValueError):
        ParallelConfig.parse(tp=4, ep=2, world=4)


def _ep_logits_worker(rank, world, port, preset, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    try:
        from metal_marlin_b200.engine.distributed import init_process_group
        from metal_marlin_b200.models.mmfp4_causal_lm import MMFP4ForCausalLM
        from metal_marlin_b200.parallel.ep import shard_transformer_ep
        r, w, dev, ctrl = init_process_group(torch.device("cpu"))
        lm = MMFP4ForCausalLM.from_config(preset, device="cpu", seed=5)
        _sharpen(lm.model)
        ids = PROMPTS[3] if rank else PROMPTS[2]          # every rank brings its own tokens (different counts)
        full = lm.forward_logits(ids)
        got = MMFP4ForCausalLM(shard_transformer_ep(lm.model, r, w, 256, mode="nccl")).forward_logits(ids)
        q.put((rank, float((got - full).abs().max() / full.abs().max())))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


@pytest.mark.parametrize("preset", ["tiny-qwen3-moe", "tiny-mla-moe"])
def test_expert_parallel_model_logits_match_unsharded(preset):
    """Expert-parallel model (experts cut to the rank's range, token rows exchanged) against the whole model on the same
    tokens; the exchange rounds expert outputs to bf16 before the weighted sum, hence a tolerance instead of equal ids."""
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_ep_logits_worker, args=(r, world, port, preset, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=600) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(v < 3e-2 for v in results.values()), results
