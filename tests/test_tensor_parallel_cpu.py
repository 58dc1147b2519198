"""Tensor-parallel sharding on CPU ranks (gloo): a 2-way sharded model must reproduce the unsharded logits.
Mirrors the reference's sharded-vs-unsharded equality suite (metal_marlin/distributed/verification.py:85-509),
but with real processes and a real collective instead of an in-process simulation."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from metal_marlin_b200.parallel.tp import even_split


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, preset, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from metal_marlin_b200.engine.session import DecodeSession, SamplingParams
        from metal_marlin_b200.models.mmfp4_causal_lm import MMFP4ForCausalLM, prefill
        from metal_marlin_b200.models.transformer import PagedKVStorage
        from metal_marlin_b200.parallel.tp import make_context, shard_transformer
        torch.manual_seed(0)
        lm = MMFP4ForCausalLM.from_config(preset, device="cpu", seed=5)
        for L in lm.model.layers:
            if L.router_w is not None:
                L.router_w.mul_(16.0)
        ctx = make_context(lm.config, torch.device("cpu"), mode="nccl")
        shard = shard_transformer(lm.model, rank, world, ctx)
        prompts = [list(range(3, 40)), list(range(50, 58))]
        bt = torch.arange(16, dtype=torch.int32).view(2, 8)

        def run(model):
            kv = PagedKVStorage(model.cfg, 16, 16, "cpu")
            if model is not lm.model and not model.cfg.is_mla:
                # GQA shards cache only their local kv heads
                import copy
                c = copy.copy(model.cfg)
                c.num_key_value_heads = model.n_kv_heads_local
                kv = PagedKVStorage(c, 16, 16, "cpu")
            lg = model.full_logits(prefill(model, kv, prompts, bt))
            sess = DecodeSession(model, kv, 2, 8, max_new_tokens=3, use_graph=False)
            sess.set_sampling([SamplingParams()] * 2)
            sess.set_state(lg.argmax(-1), [len(p) for p in prompts], bt)
            toks = [sess.step().clone() for _ in range(3)]
            return lg, torch.stack(toks)

        lg_tp, tok_tp = run(shard)
        lg_ref, tok_ref = run(lm.model)
        err = float((lg_tp - lg_ref).abs().max() / lg_ref.abs().max())
        q.put((rank, err, bool(torch.equal(tok_tp, tok_ref)), tuple(lg_tp.shape)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("preset", ["tiny-llama", "tiny-mla-moe", "tiny-qwen3-moe"])
def test_two_way_shard_matches_unsharded(preset):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, preset, q)) for r in range(2)]
    [p.start() for p in procs]
    res = [q.get(timeout=240) for _ in range(2)]
    [p.join(timeout=60) for p in procs]
    for rank, err, same_tokens, shape in res:
        assert err < 4e-2, (rank, err)
        assert same_tokens, rank
    assert res[0][3] == res[1][3]


def test_even_split_alignment():
    assert even_split(20, 8) == [(0, 2), (2, 5), (5, 7), (7, 10), (10, 12), (12, 15), (15, 17), (17, 20)]
    parts = even_split(1536, 8, 128)
    assert parts[0] == (0, 128) and parts[-1][1] == 1536 and all((b - a) % 128 == 0 and b > a for a, b in parts)
    assert even_split(154880, 8)[3] == (58080, 77440)
