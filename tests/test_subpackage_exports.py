"""Sub-package surfaces under the reference's names: speculative decoding and evaluation helpers.  Parity: reference
``metal_marlin/speculative/__init__.py`` and ``metal_marlin/eval/__init__.py`` exports."""
import os

import numpy as np
import pytest
import torch


def test_speculative_package_surface():
    from metal_marlin_b200 import spec
    for n in ("AcceptanceResult", "AcceptanceStats", "DraftOutput", "EagleHead", "EagleTreeVerifyResult", "GenerationStats",
              "MMFP4DraftModel", "MMFP4DraftModelWithTarget", "SpeculativeConfig", "StepResult", "TreeDraftOutput", "VerifyResult",
              "compute_acceptance_probabilities", "create_acceptance_report", "estimate_optimal_speculation_length", "verify_eagle_tree",
              "SpeculativeEngine", "NGramDraft", "verify_speculative"):
        assert hasattr(spec, n), n
    p = torch.tensor([[0.5, 0.5], [0.9, 0.1]])
    q = torch.tensor([[0.25, 0.75], [0.9, 0.1]])
    acc = spec.compute_acceptance_probabilities(p, q, [0, 1])
    assert torch.allclose(acc, torch.tensor([1.0, 1.0])) and float(spec.compute_acceptance_probabilities(p, q, [1, 0])[0]) == pytest.approx(2 / 3)
    assert spec.estimate_optimal_speculation_length(0.0) == 1
    assert spec.estimate_optimal_speculation_length(0.9, 0.05) > spec.estimate_optimal_speculation_length(0.5, 0.05) >= 1
    assert spec.estimate_optimal_speculation_length(0.9, 0.5) <= spec.estimate_optimal_speculation_length(0.9, 0.05)
    # tree: root -> a(0) -> b(1); root -> c(2).  The target wants token 7 then 9.
    V = 12
    root = torch.zeros(V)
    root[7] = 5
    nodes = torch.zeros(3, V)
    nodes[0, 9] = 5
    nodes[1, 3] = 5
    r = spec.verify_eagle_tree(root, nodes, tokens=[7, 9, 4], parents=[-1, 0, -1])
    assert r.accepted_path == [0, 1] and r.tokens == [7, 9, 3] and r.num_accepted == 2
    tr = spec.TokenAcceptanceTracker()
    tr.record([1, 2, 3, 4], 3)
    tr.record([1, 2, 3, 4], 1)
    rep = spec.create_acceptance_report(tr)
    assert rep["proposed"] == 8 and rep["accepted"] == 4 and rep["position_rates"][0] == 1.0 and rep["suggested_length"] >= 1
    from metal_marlin_b200.models.mmfp4_causal_lm import MMFP4ForCausalLM
    lm = MMFP4ForCausalLM.from_config("tiny-llama", device="cpu", seed=0)
    eng = spec.SpeculativeConfig(draft="ngram", num_speculative_tokens=3).build(lm)
    assert isinstance(eng, spec.SpeculativeEngine) and isinstance(eng.draft, spec.NGramDraft)


def test_eval_package_surface():
    from metal_marlin_b200 import eval as ev
    x = np.random.RandomState(0).randn(5, 7)
    assert np.allclose(ev.softmax(x).sum(-1), 1) and np.allclose(np.exp(ev.log_softmax(x)), ev.softmax(x))
    logits = torch.zeros(4, 10)
    assert ev.compute_perplexity_from_logits(logits, torch.tensor([1, 2, 3, 4])) == pytest.approx(10.0)
    kl = ev.compute_kl_divergence(torch.randn(6, 9), torch.randn(6, 9))
    same = ev.compute_kl_divergence(logits, logits)
    assert kl.kl_mean > 0 and kl.num_tokens == 6 and same.kl_mean == pytest.approx(0.0) and same.top1_agreement == 1.0
    assert ev.compute_kl_divergence_np(logits, logits) == pytest.approx(0.0)
    corpus = ev.load_wikitext2(None, max_tokens=300, vocab_size=50)
    assert len(corpus) == 300 and max(corpus) < 50

    def uniform(ids):
        return torch.zeros(len(ids), 50)
    assert ev.compute_perplexity_sliding_window(uniform, corpus, 64, 32) == pytest.approx(50.0, rel=1e-3)
    assert ev.compute_perplexity_wikitext(uniform, None, 64, 32, max_tokens=200, vocab_size=50) == pytest.approx(50.0, rel=1e-3)
    r = ev.evaluate_kl_divergence(uniform, uniform, corpus[:100], 64)
    assert r.kl_mean == pytest.approx(0.0, abs=1e-9)
    assert ev.load_tokenizer(None, 100) is not None


def test_utils_package_surface(tmp_path):
    from metal_marlin_b200 import utils as u
    assert u.calculate_matmul_flops(4, 8, 16) == 2 * 4 * 8 * 16 and u.calculate_matmul_flops(4, 8, 16, quantized=True) > 1024
    full = u.calculate_attention_flops(1, 128, 8, 64)
    assert u.calculate_attention_flops(1, 128, 8, 64, causal=True) < full and full == 4 * 8 * 128 * 128 * 64 + 5 * 8 * 128 * 128
    assert u.calculate_ffn_flops(1, 10, 64, 256, gated=True) > u.calculate_ffn_flops(1, 10, 64, 256)
    assert u.calculate_layernorm_flops(2, 3, 4) == 120 and u.calculate_embedding_flops(1, 1, 10, 10) == 0
    c = u.profile_model_flops(1, 512, 4, 1024, 8, 4096, vocab_size=32000)
    s = c.summary()
    assert s["layers"] == 5 and 0.5 < s["matmul_fraction"] < 1 and c.total_flops == sum(l.total_flops for l in c.layers)
    mem = u.get_system_memory()
    det = u.get_system_memory_detailed()
    assert mem.total_ram_gb > 0 and det.available_ram_gb <= det.total_ram_gb and u.get_metal_memory_pressure() in ("normal", "warn", "critical")
    assert isinstance(u.should_reduce_allocation(), bool)
    assert u.estimate_tensor_memory((4, 8), np.float16) == 64 and u.estimate_tensor_memory((4, 8), torch.bfloat16) == 64
    assert u.compute_optimal_batch_size([(1024, 1024)], 1.0, np.float16, 0.5) == 256
    assert u.round_up(13, 8) == 16
    a, orig = u.pad_numpy_2d(np.ones((3, 5)), rows_multiple=4, cols_multiple=8)
    t, orig_t = u.pad_torch_2d(torch.ones(3, 5), rows_multiple=4, cols_multiple=8, value=2.0)
    assert a.shape == (4, 8) and orig == (3, 5) and t.shape == (4, 8) and float(t[3, 7]) == 2.0 and orig_t == (3, 5)
    from metal_marlin_b200.formats.safetensors_io import save_file
    f1, f2 = str(tmp_path / "a.safetensors"), str(tmp_path / "b.safetensors")
    save_file({"x": torch.ones(64, 64), "y": torch.zeros(64, 64)}, f1)
    save_file({"z": torch.full((64, 64), 3.0)}, f2)
    pf = u.AdaptivePrefetcher([f1, f2], budget_bytes=64 * 64 * 4 + 8)
    got = list(pf)
    assert [sorted(b) for b in got] == [["x"], ["y"], ["z"]] and float(got[2]["z"][0, 0]) == 3.0 and len(pf.meta) == 3
    u.clear_profiles()
    u.enable_profiling()
    try:
        @u.profile_kernel("unit")
        def work():
            return sum(range(1000))
        assert work() == 499500 and work() == 499500 and u.is_profiling_enabled()
        st = u.get_profile_stats("unit")
        assert st.count == 2 and st.total_ms >= 0 and len(u.get_profile_records("unit")) == 2 and "unit" in u.get_all_profile_stats()
        lines = []
        u.print_profile_summary(lines.append)
        assert any("unit" in l for l in lines)
    finally:
        u.disable_profiling()
        u.clear_profiles()


def test_kv_package_surface():
    from metal_marlin_b200 import kv
    for n in ("BlockState", "CacheStats", "EvictionPolicy", "KVBlock", "KVBlockConfig", "MLABlock", "MLABlockAllocator", "MLACacheConfig",
              "ParityValidator", "paged_attention", "paged_attention_v1", "mla_attention", "write_kv_to_blocks", "validate_paged_v1_parity",
              "run_comprehensive_parity_suite", "compare_memory_usage", "PrefixMatch", "CachedBlock", "CacheMetrics", "QuantizedKVCache",
              "compress_kv", "decompress_kv", "hash_prefix", "hash_tokens", "PagedKVCache", "RadixPrefixCache", "KVCache", "MLAKVCache"):
        assert hasattr(kv, n), n
    res = kv.run_comprehensive_parity_suite("cpu")
    assert len(res) == 4 and all(r.passed for r in res), [r.max_abs_error for r in res]
    assert kv.ParityValidator(kv.ParityConfig(seq_len=20)).run().passed
    al = kv.BlockAllocator(4, 16)
    b = al.allocate()
    assert kv.KVBlock.of(al, b).state is kv.BlockState.ALLOCATED and kv.KVBlock.of(al, 3).state is kv.BlockState.FREE
    al.incref(b)
    assert kv.KVBlock.of(al, b).state is kv.BlockState.SHARED
    cfg = kv.KVBlockConfig(16, 8, 128, "bf16")
    assert cfg.bytes_per_token == 2 * 8 * 128 * 2 and cfg.bytes_per_block == 16 * cfg.bytes_per_token
    assert kv.KVBlockConfig(16, 8, 128, "fp8").bytes_per_token == 2 * (8 * 128 + 32)
    assert kv.MLACacheConfig().bytes_per_token == 576 * 2
    m = kv.compare_memory_usage([100, 700, 30], 4096, cfg)
    assert m["blocks"] == 7 + 44 + 2 and 0.9 < m["savings"] < 1.0 and 0 < m["internal_fragmentation"] < 0.1
    cache = kv.PagedKVCache(8, 4)
    cache.admit("a", list(range(10)))
    st = kv.CacheStats.of(cache)
    assert st.blocks == 8 and st.free == 5 and st.sequences == 1
    q = kv.QuantizedKVCache(2, 1, 2, 64, 32, dtype="fp8")
    k, v = torch.randn(1, 2, 5, 64), torch.randn(1, 2, 5, 64)
    ka, va = q.update(0, k, v)
    assert ka.shape[-2] == 5 and float((ka.float() - k).abs().max()) < 0.1 * float(k.abs().max())
    stored, sc = kv.compress_kv(k, "int8")
    assert float((kv.decompress_kv(stored, sc, "int8", torch.float32) - k).abs().max()) < 0.05 * float(k.abs().max())
    assert kv.hash_prefix([1, 2, 3]) == kv.hash_tokens([1, 2, 3])


def test_parallel_package_surface_single_process():
    from metal_marlin_b200 import parallel as par
    for n in par.__all__:
        assert getattr(par, n) is not None, n
    t = torch.arange(24.0).view(4, 6)
    assert torch.equal(par.shard_tensor(t, 1, 1, 2), t[:, 3:]) and par.shard_tensor(t, 0, 0, 4).shape == (1, 6)
    assert par.ShardSpec(0, 1, 2, unit=16).bounds(96) == (48, 96)
    x = torch.ones(3)
    assert par.all_reduce(x.clone()).tolist() == [1, 1, 1] and par.all_gather(x) is x and par.broadcast(x) is x and par.scatter(x) is x
    w, inp = torch.randn(8, 12), torch.randn(5, 12)
    ref = inp @ w.t()
    cols = [par.TensorParallelLinear(w, par.ParallelMode.COLUMN, r, 2, gather_output=False)(inp) for r in range(2)]
    assert torch.allclose(torch.cat(cols, -1), ref, atol=1e-5)
    rows = [par.TensorParallelLinear(w, par.ParallelMode.ROW, r, 2)(inp) for r in range(2)]
    assert torch.allclose(rows[0] + rows[1], ref, atol=1e-5)
    q = par.TensorParallelLinear(torch.randn(64, 256) * 0.1, par.ParallelMode.COLUMN, 1, 2, gather_output=False, quantize=True, group_size=64)
    assert q(torch.randn(3, 256)).shape == (3, 32)
    pp = par.PipelineParallel(10, par.PipelineConfig(num_stages=3), rank=1)
    assert len(pp.stages) == 3 and pp.stage_of(0) == 0 and pp.stage_of(9) == 2 and list(pp.my_layers) == list(range(*pp.stages[1]))
    devs = par.Device.discover()
    assert devs and devs[0].torch_device.type in ("cpu", "cuda")


def test_arch_blocks_carry_state_across_calls():
    from metal_marlin_b200 import arch
    torch.manual_seed(0)
    B, T, d, H = 2, 9, 64, 4
    x = torch.randn(B, T, d)
    # RWKV: one pass equals a prompt pass plus single-token steps with the carried state
    blk = arch.RWKVBlock.random(d, H, seed=1)
    full, _ = blk(x)
    y1, st = blk(x[:, :5])
    outs = [y1]
    for t in range(5, T):
        yt, st = blk(x[:, t:t + 1], st)
        outs.append(yt)
    assert torch.allclose(torch.cat(outs, 1), full, atol=1e-4) and st.wkv.shape == (B, H, d // H, d // H)
    r, k, v = (torch.randn(B, H, 16) for _ in range(3))
    w, u = torch.rand(B, H, 16), torch.randn(H, 16)
    o, s = arch.rwkv_wkv_single_token(r, k, v, w, u, torch.zeros(B, H, 16, 16))
    ob, sb = arch.rwkv_wkv_batched(r[:, None], k[:, None], v[:, None], w[:, None], u)
    assert torch.allclose(o, ob[:, 0], atol=1e-5) and torch.allclose(s, sb, atol=1e-5)
    # differential attention: shape, causality
    da = arch.DifferentialAttention.random(arch.parse_diff_transformer_config({"hidden_size": d, "num_attention_heads": 4}, layer_idx=2))
    ya = da(x)
    x2 = x.clone()
    x2[:, -1] += 1.0
    assert ya.shape == x.shape and torch.allclose(da(x2)[:, :-1], ya[:, :-1], atol=1e-5) and 0.2 < da.cfg.lambda_init < 0.8
    # hybrid stacks: pieces with carried states equal one pass, for every family
    for kind, kw in (("jamba", {"attn_period": 2, "attn_offset": 1}), ("rwkv", {}), ("mamba", {}), ("attention", {}), ("zamba", {"shared_every": 2})):
        cfg = arch.build_hybrid_config(kind, d, 4, num_heads=H, **kw)
        model = arch.HybridModelBuilder(cfg).build(seed=3)
        whole, states = model(x)
        a, st = model(x[:, :4])
        b, st = model(x[:, 4:], st)
        assert torch.allclose(torch.cat([a, b], 1), whole, atol=2e-4), kind
        assert len(states) == 4 and len(model.state_types()) == 4
    assert arch.StateType.KV_CACHE in arch.HybridModelBuilder(arch.build_hybrid_config("jamba", d, 4, H, attn_period=2, attn_offset=1)).build().state_types()
    assert arch.MarlinMambaBlock is arch.MambaBlock and arch.MambaLayerConfig is arch.MambaConfig


def test_inference_and_serving_package_surfaces():
    from metal_marlin_b200 import inference as inf
    from metal_marlin_b200 import serving as srv
    for n in inf.__all__:
        assert getattr(inf, n) is not None, n
    for n in srv.__all__:
        assert getattr(srv, n) is not None, n
    assert inf.get_device("cpu") == "cpu" and inf.get_device() in ("cpu",) or inf.get_device().startswith("cuda")
    from metal_marlin_b200.compat_api import pack_fp4_weights
    w = torch.randn(128, 24) * 0.1
    p, s, _m = pack_fp4_weights(w, 64, output_backend="torch")
    d = inf.dequantize_fp4_torch(p, s)
    assert d.shape == (128, 24) and float((d - w).abs().max()) < 0.26 * float(w.abs().max())
    hid = torch.randn(2, 3, 16)
    r = inf.batched_kv_projection(hid, torch.randn(8, 16), torch.randn(8, 16), 2, 4)
    assert r.keys.shape == (2, 3, 2, 4) and r.values.shape == (2, 3, 2, 4) and r.num_tokens == 6
    pipe = inf.MMFP4Pipeline.from_config("tiny-llama", device="cpu")
    info = inf.ModelInfo.of(pipe)
    assert info.num_layers == 2 and info.attention == "gqa" and isinstance(inf.chat(pipe, [{"role": "user", "content": "hi"}], max_new_tokens=2), str)
    from metal_marlin_b200.kv import PagedKVCache
    c = PagedKVCache(8, 4)
    c.admit("s", list(range(6)))
    reg = srv.KVRegion.of(c, "s")
    assert reg.num_tokens == 6 and len(reg.blocks) == 2 and len(reg.slots()) == 6 and srv.KVCacheManager is PagedKVCache


def test_layer_objects_moe_mla_mixed_precision():
    from metal_marlin_b200 import layers
    torch.manual_seed(0)
    E, H, I, T, k = 8, 128, 64, 6, 2
    router = torch.randn(E, H) * 0.1
    gate, up, down = torch.randn(E, I, H) * 0.1, torch.randn(E, I, H) * 0.1, torch.randn(E, H, I) * 0.1
    shared = (torch.randn(1, I, H) * 0.1, torch.randn(1, I, H) * 0.1, torch.randn(1, H, I) * 0.1)
    moe = layers.MMFP4MoE.from_float(router, gate, up, down, top_k=k, shared=shared, group_size=64)
    x = torch.randn(T, H)
    y = moe(x)
    ids, wts = moe.route(x.bfloat16())
    gu, dn = moe.gate_up.dequantize(torch.float32), moe.down.dequantize(torch.float32)

    def expert(e, v):
        h = gu[e] @ v
        return dn[e] @ (F_silu(h[:I]) * h[I:])
    F_silu = torch.nn.functional.silu
    xb = x.bfloat16().float()
    ref = torch.stack([sum(float(wts[t, j]) * expert(int(ids[t, j]), xb[t]) for j in range(k)) + expert(E, xb[t]) for t in range(T)])
    assert y.shape == x.shape and float((y - ref).abs().max()) < 0.05 * float(ref.abs().max()) + 1e-3
    assert layers.MMFP4FusedMoE is layers.MMFP4MoE and layers.MMFP4MTPHead is layers.GLMMTPHead
    # MLA: a prompt pass plus single-token steps over the latent cache equals one pass over the whole sequence
    mla = layers.MMFP4MLA.from_float(hidden=128, num_heads=4, q_lora_rank=64, kv_lora_rank=64, qk_nope_head_dim=32, qk_rope_head_dim=16,
                                     v_head_dim=32, seed=1)
    xs = torch.randn(2, 7, 128)
    whole = mla(xs)
    cache = mla.new_cache(batch=2, max_seq_len=16)
    parts = [mla(xs[:, :4], cache=cache)] + [mla(xs[:, t:t + 1], cache=cache) for t in range(4, 7)]
    assert whole.shape == xs.shape and cache.seq_len == 7
    assert float((torch.cat(parts, 1) - whole).abs().max()) < 0.03 * float(whole.abs().max()) + 1e-3
    x2 = xs.clone()
    x2[:, -1] += 1
    assert torch.allclose(mla(x2)[:, :-1], whole[:, :-1], atol=1e-3)          # causal
    # precision policy picks the storage
    w = torch.randn(64, 128) * 0.1
    for prec, tol in (("fp4", 0.3), ("int8", 0.03), ("bf16", 0.02)):
        lin = layers.MixedPrecisionLinear(w, prec, 64)
        out = lin(x[:, :128])
        assert float((out - x[:, :128] @ w.t()).abs().max()) < tol * float((x[:, :128] @ w.t()).abs().max()) + 1e-2, prec
    assert layers.MixedPrecisionLinear.for_tensor("model.layers.0.input_layernorm.weight", w).format == "keep"
    assert layers.MixedPrecisionLinear.for_tensor("model.layers.0.self_attn.q_proj.weight", w, "quality").format == "int8"
    # vectorised verification: a draft equal to the target's arg-max with one-hot distributions is accepted whole
    V, K = 11, 3
    tgt = torch.zeros(1, K + 1, V)
    tgt[0, torch.arange(K + 1), torch.tensor([1, 2, 3, 4])] = 1.0
    dr = torch.zeros(1, K, V)
    dr[0, torch.arange(K), torch.tensor([1, 2, 3])] = 1.0
    toks, acc = layers.verify_kernel(tgt, dr, torch.tensor([[1, 2, 3]]), generator=torch.Generator().manual_seed(0))
    assert int(acc[0]) == 3 and toks[0].tolist() == [1, 2, 3, 4]


def test_moe_and_memory_package_surfaces(tmp_path):
    from metal_marlin_b200 import layers, memory, moe
    from metal_marlin_b200.models.config import get_preset
    ids = torch.tensor([[0, 3], [3, 1], [2, 0], [3, 2]], dtype=torch.int32)
    res = moe.GPUExpertGrouping(4, token_tile=2).group(ids)
    assert int(res.num_tiles) >= 4 and torch.equal(res.order.long()[res.inverse.long()], torch.arange(8))
    order, offsets, inv = moe.group_tokens_by_expert_auto(ids, 4)
    assert offsets.tolist() == [0, 2, 3, 5, 8] and moe.group_tokens_by_expert_full_gpu(ids, 4).num_tokens == 4
    torch.manual_seed(0)
    lay = layers.MMFP4MoE.from_float(torch.randn(4, 64) * 0.1, torch.randn(4, 64, 64) * 0.1, torch.randn(4, 64, 64) * 0.1,
                                     torch.randn(4, 64, 64) * 0.1, top_k=2, group_size=64)
    disp = moe.MoEDispatcher(lay)
    x = torch.randn(5, 64)
    assert torch.allclose(disp(x), lay(x), atol=1e-5) and int(disp.tracker.counts.sum()) == 10 and moe.FusedMoEDispatcher is moe.MoEDispatcher
    # memory planning for the GLM-4.7-Flash configuration
    cfg = get_preset("glm-4.7-flash")
    mgr = memory.MMFP4MemoryManager(cfg, limit_bytes=180 << 30)
    plan = mgr.plan()
    st = plan["stats"]
    assert plan["fits_entirely"] and 12e9 < st.weight_bytes + st.resident_expert_bytes < 22e9 and st.kv_tokens_that_fit > 1_000_000
    small = memory.MMFP4MemoryManager(cfg, limit_bytes=8 << 30).plan()
    assert not small["fits_entirely"] and small["stats"].offloaded_expert_bytes > 0 and any(not e.resident for e in small["experts"])
    r = memory.MLACompressionRatio.of(cfg)
    assert r.latent_bytes_per_token == 576 * 2 and r.ratio > 15
    assert mgr.kv_bytes_per_token() == 576 * 2 * cfg.num_hidden_layers
    # compaction wrapper and memory-mapped weights
    arena = memory.Arena(4096, "cpu", alignment=64)
    a, b, c = (arena.alloc((512,), torch.uint8) for _ in range(3))
    c.fill_(7)
    off_c = arena.offset_of(c)
    arena.free(a)
    arena.free(b)
    moved = {}
    comp = memory.MemoryCompactor(arena, memory.CompactionConfig(0.0, 0.0), on_moved=lambda o, n: moved.update({o: n}))
    assert comp.maybe_compact(force=True) >= 1 and moved[off_c] < off_c and comp.stats.runs == 1
    from metal_marlin_b200.formats.safetensors_io import save_file
    d = tmp_path / "ck"
    d.mkdir()
    save_file({"model.layers.0.w": torch.ones(4, 4), "model.layers.1.w": torch.zeros(2, 2), "model.norm.weight": torch.ones(4)}, str(d / "model.safetensors"))
    mm = memory.MMAPWeightManager(str(d))
    assert sorted(mm.names())[0] == "model.layers.0.w" and float(mm.get("model.layers.0.w").sum()) == 16 and list(mm.layer(1)) == ["model.layers.1.w"]
    assert mm.stats.loads == 2 and mm.stats.bytes_loaded == 64 + 16 and memory.CUDAPinnedPool is memory.PinnedPool
    mm.close()
    pb = memory.PooledBuffer(torch.empty(8))
    pb.touch()
    assert pb.use_count == 1


def test_trellis_package_surface():
    from metal_marlin_b200 import trellis as tr
    for n in tr.__all__:
        assert getattr(tr, n) is not None, n
    torch.manual_seed(0)
    codes = torch.randint(0, 8, (32, 48), dtype=torch.uint8)
    blob = tr.pack_indices(codes, 3)
    assert blob.numel() == tr.compute_packed_size(32, 48, 3) and int(blob[0]) == 3
    assert torch.equal(tr.unpack_indices(blob, 32, 48), codes) and torch.equal(tr.unpack_trellis_indices(tr.pack_trellis_indices(codes, 3), 32, 48), codes)
    assert 3.5 < tr.compute_compression_ratio(4096, 4096, 4) < 4.0 and tr.compute_compression_ratio(4096, 4096, 2) > 7
    w = torch.randn(64, 128) * 0.05
    lin = tr.TrellisLinear.from_float(w, 4, 64)
    deq = tr.dequantize_trellis_weight(lin, torch.float32)
    assert float((deq - w).abs().max()) < 0.25 * float(w.abs().max())
    again = tr.dispatch_trellis_dequant(lin.codes, lin.scales, lin.su, lin.sv, 64, 128, 4, 64).float()
    assert torch.allclose(again, deq, atol=1e-2)
    x = torch.randn(3, 128)
    assert float((tr.dispatch_gemm_trellis_auto(x, lin).float() - x.bfloat16().float() @ deq.t()).abs().max()) < 0.05
    assert torch.equal(tr.dispatch_sign_flips(torch.ones(2, 4), torch.tensor([1.0, -1, 1, -1])), torch.tensor([[1.0, -1, 1, -1]] * 2))
    # dense MLP and a mixed-bit MoE MLP against their de-quantized restatement
    H, I, E = 128, 64, 4
    mk = lambda bits, seed: tr.TrellisDenseMLP.from_float(*(torch.randn(*s, generator=torch.Generator().manual_seed(seed + i)) * 0.1
                                                          for i, s in enumerate(((I, H), (I, H), (H, I)))), bits=bits, group_size=64)
    mlp = mk(4, 0)

    def ref_mlp(m, v):
        g, u, d = (t.dequantize(torch.float32) for t in (m.gate, m.up, m.down))
        return (torch.nn.functional.silu(v @ g.t()) * (v @ u.t())) @ d.t()
    xb = x.bfloat16().float()
    assert float((mlp(x).float() - ref_mlp(mlp, xb)).abs().max()) < 0.05 * float(ref_mlp(mlp, xb).abs().max()) + 1e-3
    experts = [mk(b, 10 * e) for e, b in enumerate((2, 3, 4, 4))]
    moe = tr.TrellisMoEMLP(torch.randn(E, H) * 0.1, experts, tr.MoEConfig(E, 2, H, I, num_shared_experts=1), shared=[mk(4, 99)])
    tr.reset_mixed_bpw_stats()
    y = tr.dispatch_mixed_bpw_moe(x, moe)
    ids, wts = moe.route(x.bfloat16())
    ref = torch.stack([sum(float(wts[t, j]) * ref_mlp(experts[int(ids[t, j])], xb[t:t + 1])[0] for j in range(2)) + ref_mlp(moe.shared[0], xb[t:t + 1])[0]
                       for t in range(3)])
    assert float((y.float() - ref).abs().max()) < 0.06 * float(ref.abs().max()) + 1e-3
    st = tr.get_mixed_bpw_stats()
    assert st["calls"] == 1 and st["tokens"] == 3 and sum(st["by_bits"].values()) == 6
    # MLA attention over trellis projections, inside a decoder layer, with the compressed latent cache
    cfg = tr.TrellisMLAConfig(H, 4, 64, 64, 32, 16, 32)
    g = torch.Generator().manual_seed(5)
    rn = lambda *s: torch.randn(*s, generator=g) * 0.05
    state = {"q_a_proj": rn(64, H), "q_a_layernorm": torch.ones(64), "q_b_proj": rn(4 * 48, 64), "kv_a_proj_with_mqa": rn(64 + 16, H),
             "kv_a_layernorm": torch.ones(64), "kv_b_proj": rn(4 * 64, 64), "o_proj": rn(H, 4 * 32)}
    attn = tr.TrellisMLAttention(cfg, tr.create_mla_projections(cfg, state, bits=4, group_size=32))
    layer = tr.TrellisDecoderLayer(attn, mlp, torch.ones(H), torch.ones(H))
    xs = torch.randn(1, 6, H)
    whole = layer(xs)
    cache = tr.CompressedKVCache(1, 64, 16, 1, 16, dtype="bf16")
    parts = torch.cat([layer(xs[:, :4], cache=cache), layer(xs[:, 4:5], cache=cache), layer(xs[:, 5:], cache=cache)], 1)
    assert float((parts - whole).abs().max()) < 0.03 * float(whole.abs().max()) + 1e-3 and cache.seq_len == 6
    with pytest.raises(ValueError):
        tr.TrellisMLAttention(cfg, {"kv_a": None})
    assert tr.MixedBPWAutoTuner.__name__ == "KernelAutoTuner" and tr.TrellisModelWrapper is tr.TrellisForCausalLM


# ------------------------------------------------------------------------------------------------ quantization / calibration names
REFERENCE_QUANTIZATION = [
    "BartowskiCalibration", "CalibrationBatch", "CalibrationDataset", "CalibrationHooks", "CalibrationStreamer", "EXL3QuantResult",
    "EXL3Quantizer", "EXL3QuantizerPipeline", "GQACalibrationHooks", "LayerInfo", "LayerStreamer", "LayerWeights", "StreamingHessianCollector",
    "StreamingQuantizer", "TrellisCodebook", "TrellisTile", "analyze_layer_sensitivity", "blockwise_hadamard", "collect_all_hessians_streaming",
    "collect_layer_hessian", "compute_model_sensitivity_profile", "compute_quantization_error", "compute_tile_scales", "copy_non_linear_tensors",
    "ldl_solve", "ldlq_quantize_layer", "ldlq_quantize_layer_core", "load_sensitivity_profile", "pack_indices", "preprocess_hessian_exl3",
    "quantize_model_exl3", "quantize_model_streaming", "quantize_tiles_parallel", "recommend_quantization", "rotate_weights_exl3", "save_exl3_layer",
    "save_sensitivity_profile", "sensitivity_to_config", "tensor_core_perm", "tensor_core_perm_i", "unrotate_weights_exl3",
]


def test_quant_package_names_resolve():
    import metal_marlin_b200.quant as q
    for n in REFERENCE_QUANTIZATION + ["gptq_quantize", "mr_gptq_quantize", "ldlq_quantize", "quantize_checkpoint", "allocate_bits", "convert_model"]:
        assert getattr(q, n) is not None, n
    assert set(REFERENCE_QUANTIZATION) <= set(q.__all__)


def test_exl3_pieces_numerics(tmp_path):
    import metal_marlin_b200.quant as q
    torch.manual_seed(0)
    w = torch.randn(64, 256)
    x = torch.randn(512, 256)
    H = q.preprocess_hessian_exl3(q.collect_layer_hessian(x), damp=0.01)
    assert torch.allclose(H, H.t()) and torch.linalg.eigvalsh(H.double()).min() > 0
    # rotation is an orthonormal involution and keeps w @ x^T when x is rotated too
    wr = q.rotate_weights_exl3(w, 128)
    assert torch.allclose(q.unrotate_weights_exl3(wr, 128), w, atol=1e-4)
    assert torch.allclose(wr @ q.blockwise_hadamard(x, 128).t(), w @ x.t(), atol=1e-2)
    L, D = q.ldl_solve(H.double(), 16)
    assert L.shape == H.shape
    r4 = q.EXL3Quantizer(bits=4).quantize_layer(w, H)
    r2 = q.EXL3Quantizer(bits=2).quantize_layer(w, H)
    assert r4.bits == 4 and r4.dequantized.shape == w.shape and r4.proxy_error < r2.proxy_error
    err = q.compute_quantization_error(w, r4.dequantized, H)
    assert err["relative"] < 0.2 and err["proxy"] > 0
    # fragment-order permutation and its inverse
    p, pi = q.tensor_core_perm(), q.tensor_core_perm_i()
    assert sorted(p.tolist()) == list(range(256)) and torch.equal(p[pi], torch.arange(256))
    tile = torch.arange(256.).reshape(16, 16)
    assert torch.equal(q.apply_tensor_core_perm_i(q.apply_tensor_core_perm(tile)), tile)
    cb = q.TrellisCodebook(3)
    codes = cb.encode(cb.values + 1e-4)
    assert codes.tolist() == list(range(8)) and torch.equal(cb.decode(codes), cb.values)
    d = q.save_exl3_layer({"model.layers.0.mlp.up_proj.weight": r4.weight}, str(tmp_path), 0)
    assert os.path.isfile(os.path.join(d, "index.json")) and os.path.isfile(os.path.join(d, "tensor_0000.safetensors"))


def test_sensitivity_profile_roundtrip_and_recommendation(tmp_path):
    import metal_marlin_b200.quant as q
    torch.manual_seed(1)
    tensors = {"a": torch.randn(32, 128), "b": torch.randn(32, 128) * torch.linspace(0.1, 8, 128)}
    prof = q.compute_model_sensitivity_profile(tensors, bit_choices=(2, 3, 4, 6))
    for v in prof.values():
        e = v["error_by_bits"]
        assert e[2] > e[3] > e[4] > e[6]
    path = str(tmp_path / "p" / "profile.json")
    q.save_sensitivity_profile(prof, path)
    assert q.load_sensitivity_profile(path) == prof
    rec = q.recommend_quantization(prof, target_bpw=3.5)
    assert set(rec) == {"a", "b"} and sum(rec.values()) / 2 <= 3.5 + 1e-6
    cfg = q.sensitivity_to_config(prof, 3.5)
    assert cfg["a"]["format"] == "trellis" and cfg["a"]["bits"] == rec["a"]


def test_layer_streamer_calibration_hooks_and_streaming_quantizer(tmp_path):
    import metal_marlin_b200.quant as q
    from metal_marlin_b200.models.mmfp4_causal_lm import MMFP4ForCausalLM
    from metal_marlin_b200.formats.safetensors_io import save_file
    from metal_marlin_b200.models.config import get_preset
    cfg = get_preset("tiny-llama")
    src = str(tmp_path / "hf")
    os.makedirs(src)
    save_file(q.random_hf_state(cfg, 0), os.path.join(src, "model.safetensors"), metadata={"format": "pt"})
    cfg.save_pretrained(src)
    st = q.LayerStreamer(src)
    infos = st.layer_infos()
    assert len(infos) >= 1 and infos[0].nbytes > 0
    layers = list(st)
    assert [l.index for l in layers] == list(range(len(infos))) and set(layers[0].tensors) == set(infos[0].tensor_names)
    assert any("embed" in k for k in st.non_layer_tensors())
    res = q.quantize_model_streaming(src, str(tmp_path / "q"), fmt="mmfp4", method="rtn")
    assert res.layers == len(infos) and res.tensors > 0
    n = q.copy_non_linear_tensors(str(tmp_path / "q"), str(tmp_path / "base.safetensors"))
    assert n > 0
    lm = MMFP4ForCausalLM.from_pretrained(str(tmp_path / "q"), "cpu")
    ds = q.CalibrationDataset("synthetic", vocab_size=lm.config.vocab_size, num_samples=2, seq_len=16)
    batches = list(q.CalibrationStreamer(ds, batch_size=2))
    assert len(batches) == 1 and batches[0].input_ids.shape == (2, 16)
    with q.CalibrationHooks() as h:
        with torch.no_grad():
            lm.forward_logits(ds[0])
    names = h.collector.names()
    assert any(n.endswith("q_proj.weight") for n in names) and h.collector.n[names[0]] == 16


def test_viterbi_tile_search_is_optimal():
    import itertools
    import metal_marlin_b200.quant as q
    cb = q.TrellisCodebook(2)
    torch.manual_seed(3)
    x = torch.randn(6)
    g = cb.values.double()
    for lam in (0.0, 0.4, 2.0):
        idx, deq = q.quantize_tile_viterbi(x, cb, 0.9, transition_penalty=lam)
        cost = lambda s: float(((x.double() / 0.9 - g[list(s)]) ** 2).sum()) + lam * sum(abs(a - b) for a, b in zip(s, s[1:]))   # noqa: E731
        best = min(itertools.product(range(4), repeat=6), key=cost)
        assert abs(cost(tuple(idx.tolist())) - cost(best)) < 1e-9
        assert torch.allclose(deq, (g[idx.long()] * 0.9).float())
    assert torch.equal(q.quantize_tile_viterbi(x, cb, 0.9)[0], cb.encode(x / 0.9))


def test_exl3_config_and_hessian_manager(tmp_path):
    import json
    import torch.nn as nn
    import metal_marlin_b200.quant as q
    torch.manual_seed(0)
    res = [q.EXL3Quantizer(bits=b).quantize_layer(torch.randn(32, 128), None) for b in (3, 4, 4)]
    path = q.write_exl3_config(str(tmp_path / "out"), 4, 128, res)
    with open(path) as f:
        cfg = json.load(f)
    assert cfg["quantization_config"]["format"] == "exl3_4bit" and cfg["quantization_stats"]["layers_quantized"] == 3
    assert cfg["quantization_stats"]["bits_histogram"] == {"3": 1, "4": 2} and cfg["quantization_stats"]["avg_reconstruction_mse"] > 0
    hm = q.HessianManager(default_damp=0.1)
    hm.register_layer("a", 8)
    x = torch.randn(20, 8)
    hm.accumulate_layer("a", x[:12])
    hm.accumulate_layer("a", x[12:].numpy())
    H = x.t() @ x / 20
    assert torch.allclose(hm.get_hessian("a", damp=0.0), H, atol=1e-5) and hm.get_sample_counts() == {"a": 20}
    assert torch.allclose(hm.get_hessian("a"), H + torch.eye(8) * 0.1 * torch.diag(H).mean(), atol=1e-5)
    with pytest.raises(KeyError):
        hm.accumulate_layer("b", x)
    with pytest.raises(ValueError):
        hm.accumulate_layer("a", torch.randn(3, 7))
    hm.reset_layer("a")
    assert hm.get_sample_counts() == {"a": 0} and torch.allclose(hm.get_hessian("a"), torch.eye(8) * 0.1)
    model = nn.Sequential(nn.Linear(8, 16), nn.ReLU(), nn.Linear(16, 4))
    assert hm.attach(model, prefix="m.") == 2 and hm.num_layers == 3 and "m.2" in hm.layer_names
    model(x)
    hm.remove_hooks()
    model(x)
    assert hm.get_sample_counts()["m.0"] == 20 and set(hm.get_all_hessians()) == {"a", "m.0", "m.2"}
    hm.unregister_layer("a")
    hm.reset_all()
    assert hm.layer_names == ["m.0", "m.2"] and hm.get_sample_counts()["m.2"] == 0


def test_remaining_reference_subpackage_names():
    import importlib
    want = {"layers": ["MarlinLinear"], "inference": ["GenerationConfig", "MetalMarlinModel", "ModelConfig"],
            "quant": ["write_exl3_config", "quantize_tile_viterbi", "AdaptiveQuantizer", "AdaptiveQuantResult", "LayerBudget", "ModelBudgetAllocation",
                      "compute_moe_expert_sensitivity", "HessianManager", "LayerSensitivity"],
            "moe": ["compute_expert_load", "compute_load_balancing_loss", "gather_for_experts", "scatter_expert_outputs"],
            "trellis": ["TrellisWeight", "TrellisModelLoader"],
            "serving": ["SchedulerConfig", "ContinuousSchedulerConfig", "PreemptionPolicy", "RequestPriority", "RequestState", "ModelConfig", "_kv_sharing"]}
    for pkg, names in want.items():
        mod = importlib.import_module("metal_marlin_b200." + pkg)
        for n in names:
            assert getattr(mod, n) is not None, (pkg, n)
            assert n in mod.__all__, (pkg, n)
    import metal_marlin_b200.serving as s
    sharing = s._kv_sharing()
    assert sharing.create_region("a", [1, 2, 3, 4, 5]).num_tokens == 5 and sharing.attach("b", [1, 2, 3, 4, 5]) is not None
    from metal_marlin_b200.kv.paged import PagedKVCache

    class Holder:
        cache = PagedKVCache(8, 16)
    assert s._kv_sharing(Holder()).cache is Holder.cache


def test_every_reference_subpackage_name_resolves():
    """``tests/data/reference_subpackage_exports.json``: for each sub-package of the reference, the names in its ``__all__`` and the
    sub-package of this framework that serves them."""
    import importlib
    import json
    with open(os.path.join(os.path.dirname(__file__), "data", "reference_subpackage_exports.json")) as f:
        table = json.load(f)
    missing, total = [], 0
    for ref_pkg, entry in table.items():
        mod = importlib.import_module("metal_marlin_b200." + entry["package"])
        for n in entry["names"]:
            total += 1
            try:
                if getattr(mod, n) is None and n not in ("_HAS_SAFETENSORS",):
                    missing.append((ref_pkg, n))
            except Exception as e:          # an AttributeError or a failing lazy import
                missing.append((ref_pkg, n, repr(e)[:80]))
    assert total > 400 and not missing, missing
