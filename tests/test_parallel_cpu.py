"""Mesh, expert parallelism, pipeline parallelism and ring attention on CPU ranks (gloo, real processes); each must
reproduce the single-process result (reference: metal_marlin/distributed/verification.py)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from metal_marlin_b200.parallel.mesh import DeviceMesh, MeshShape, plan_mesh
from metal_marlin_b200.parallel.pp import stage_layers


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def test_mesh_coordinates_and_planning():
    m = DeviceMesh(MeshShape(dp=2, pp=2, tp=2), rank=5, create_groups=False)
    assert m.coords() == (1, 0, 1) and m.rank_of(1, 0, 1) == 5
    assert m.group_ranks("tp") == [4, 5] and m.group_ranks("pp") == [5, 7] and m.group_ranks("dp") == [1, 5]
    assert m.pp_neighbours() == (None, 7)
    assert len(m.all_groups("tp")) == 4 and sorted(sum(m.all_groups("dp"), [])) == list(range(8))
    assert plan_mesh(8, 20e9) == MeshShape(8, 1, 1)                 # fits one GPU: replicas
    assert plan_mesh(8, 500e9) == MeshShape(2, 1, 4)                # needs 4 GPUs of 180 GB
    assert plan_mesh(8, 20e9, prefer="tp") == MeshShape(1, 1, 8)
    assert stage_layers(10, 4) == [(0, 3), (3, 6), (6, 8), (8, 10)]


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from metal_marlin_b200 import ops
        from metal_marlin_b200.models.mmfp4_causal_lm import MMFP4ForCausalLM
        from metal_marlin_b200.models.transformer import BatchMeta
        from metal_marlin_b200.parallel.cp import ring_attention
        from metal_marlin_b200.parallel.ep import ExpertParallelMoE
        from metal_marlin_b200.parallel.pp import PipelineStage, pipeline_prefill
        res = {}
        mesh = DeviceMesh(MeshShape(dp=1, pp=1, tp=world))
        res["mesh"] = mesh.group_ranks("tp") == list(range(world)) and mesh.group("tp") is not None
        lm = MMFP4ForCausalLM.from_config("tiny-mla-moe", device="cpu", seed=5)
        cfg = lm.config
        L = next(l for l in lm.model.layers if l.router_w is not None)
        torch.manual_seed(1)
        T = 6
        x = (torch.randn(T, cfg.hidden_size) * 0.5).to(torch.bfloat16)
        ids = torch.stack([torch.randperm(cfg.num_experts)[: cfg.num_experts_per_tok] for _ in range(T)]).to(torch.int32)
        wts = torch.rand(T, cfg.num_experts_per_tok)
        full = ops.moe_forward(x, L.gate_up_bank, L.down_bank, ids, wts, n_shared=cfg.n_shared_experts, shared_base=cfg.num_experts,
                               norm_w=L.post_norm).float()
        ep = ExpertParallelMoE(L.gate_up_bank, L.down_bank, cfg.num_experts, cfg.n_shared_experts, rank, world)
        got = ep.forward_replicated(x, ids, wts, norm_w=L.post_norm).float()
        res["ep_replicated"] = float((got - full).abs().max() / full.abs().max())
        # dispatch regime: each rank owns half of the tokens; shared experts are added by the owner of the tokens
        half = slice(rank * T // world, (rank + 1) * T // world)
        routed = ops.moe_forward(x, L.gate_up_bank, L.down_bank, ids, wts, n_shared=0, shared_base=cfg.num_experts, norm_w=L.post_norm).float()
        got_d = ep.forward_dispatch(x[half], ids[half], wts[half], norm_w=L.post_norm).float()
        res["ep_dispatch"] = float((got_d - routed[half]).abs().max() / routed.abs().max())
        # the fused entry point falls back to the collective path off the GPU (and adds what the caller passes)
        got_f = ep.forward_fused(None, x[half], ids[half], wts[half], norm_w=L.post_norm, add0=x[half]).float()
        want_f = routed[half] + x[half].float()
        res["ep_fused_cpu"] = float((got_f - want_f).abs().max() / want_f.abs().max())
        # pipeline: 2 stages vs the whole model
        toks = list(range(3, 19))
        ref_logits = lm.forward_logits(toks)
        stage = PipelineStage(lm.model, rank, world, rank - 1 if rank else None, rank + 1 if rank + 1 < world else None)
        nb = 2
        kv = lm.new_cache(nb, 16)
        pos = torch.arange(len(toks), dtype=torch.int32)
        meta = BatchMeta(positions=pos, slots=pos.long(), block_tables=torch.arange(nb, dtype=torch.int32).view(1, nb),
                         ctx_lens=torch.tensor([len(toks)], dtype=torch.int32), decode=False, cu_seqlens=[0, len(toks)],
                         ctx_lens_host=[len(toks)])
        outs = pipeline_prefill(stage, [(torch.tensor(toks), kv, meta, None)])
        if stage.is_last:
            res["pp"] = float((outs[0] - ref_logits).abs().max() / ref_logits.abs().max())
        # several micro-batches (different sequences) with overlapped hand-overs: receives posted ahead, sends in the background;
        # the same answer as with blocking hand-overs, micro-batch by micro-batch
        seqs = [list(range(3 + i, 12 + 2 * i)) for i in range(4)]
        def mbs():
            out = []
            for s_ in seqs:
                kv_i = lm.new_cache(2, 16)
                p_i = torch.arange(len(s_), dtype=torch.int32)
                out.append((torch.tensor(s_), kv_i, BatchMeta(positions=p_i, slots=p_i.long(), block_tables=torch.arange(2, dtype=torch.int32).view(1, 2),
                                                              ctx_lens=torch.tensor([len(s_)], dtype=torch.int32), decode=False,
                                                              cu_seqlens=[0, len(s_)], ctx_lens_host=[len(s_)]), None))
            return out
        a = pipeline_prefill(stage, mbs(), overlap=True, max_inflight_sends=1)
        b = pipeline_prefill(stage, mbs(), overlap=False)
        if stage.is_last:
            res["pp_overlap"] = max(float((x - y).abs().max()) for x, y in zip(a, b))
            res["pp_multi"] = max(float((x - lm.forward_logits(s_)).abs().max() / x.abs().max()) for x, s_ in zip(a, seqs))
        # ring attention vs dense causal attention
        torch.manual_seed(2)
        S = 8
        qf, kf, vf = torch.randn(1, 4, S * world, 16), torch.randn(1, 2, S * world, 16), torch.randn(1, 2, S * world, 16)
        dense = torch.nn.functional.scaled_dot_product_attention(qf, kf.repeat_interleave(2, 1), vf.repeat_interleave(2, 1), is_causal=True)
        sl = slice(rank * S, (rank + 1) * S)
        ring = ring_attention(qf[:, :, sl], kf[:, :, sl], vf[:, :, sl])
        res["cp"] = float((ring - dense[:, :, sl]).abs().max())
        q.put((rank, res))
    finally:
        dist.destroy_process_group()


def test_ep_pp_cp_on_two_cpu_ranks():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=300) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for r in range(world):
        res = results[r]
        assert res["mesh"]
        assert res["ep_replicated"] < 2e-2, res
        assert res["ep_dispatch"] < 2e-2, res
        assert res["ep_fused_cpu"] < 3e-2, res
        assert res["cp"] < 1e-4, res
    assert results[world - 1]["pp"] < 1e-2, results
    assert results[world - 1]["pp_overlap"] == 0.0 and results[world - 1]["pp_multi"] < 1e-2, results


def test_ep_exchange_layout_and_descriptors():
    """Buffer layout of the expert-parallel exchange: regions do not overlap, every rank's tables point into the peers'
    buffers at the same offsets, descriptors have the lengths the kernels expect."""
    from metal_marlin_b200.parallel.ep import EPExchange
    ep, H, T, k = 4, 64, 6, 2
    lay = EPExchange.layout(ep, T * k, H)
    assert EPExchange.OFF_META <= lay["meta"] < lay["recv_x"] < lay["ret_y"] < lay["bytes"]
    assert lay["recv_x"] - lay["meta"] >= ep * T * k * 8 and lay["ret_y"] - lay["recv_x"] >= ep * T * k * H * 2
    assert lay["recv_x"] % 256 == 0 and lay["ret_y"] % 256 == 0
    exs = EPExchange.emulated(ep, H, T, k, "cpu")
    for r, ex in enumerate(exs):
        assert ex.rank == r and ex.cap == T * k and ex.recv_x.shape == (ep * T * k, H) and ex.ret_y.shape == (T * k, H)
        assert [len(d) for d in (ex.desc_dispatch, ex.desc_recv, ex.desc_signal, ex.desc_combine)] == [8, 6, 2, 4]
        tbl = ex._tbl
        for d in range(ep):
            base = exs[d].local.data_ptr()
            assert int(tbl[0, d]) == base + lay["recv_x"] and int(tbl[1, d]) == base + lay["meta"]
            assert int(tbl[3, d]) == base + EPExchange.OFF_FLAGS + 4 * r              # dispatch flag [0][r] on rank d
            assert int(tbl[5, d]) == base + EPExchange.OFF_FLAGS + 4 * (ep + r)       # return flag [1][r] on rank d
        ex.begin()
        assert int(ex.step.item()) == 1 and ex.check() == 0
