"""Smaller components: tiered / radix prompt cache, request batcher, KV sharing, W&B shim, benchmark report, NeMo
conversion, additional GGUF block types, early exit.  Reference: tests/test_prompt_cache.py, tests/test_request_batcher.py,
tests/test_kv_sharing.py, tests/test_early_exit.py, tests/test_gguf_loader.py."""
import asyncio
import io
import json
import tarfile

import numpy as np
import torch
import yaml

from metal_marlin_b200.kv.paged import PagedKVCache
from metal_marlin_b200.kv.prompt_cache import PrefixCacheConfig, RadixPrefixCache, StorageTier, TieredPrefixCache


def _kv_blocks(n, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [torch.randn(2, 16, 4, 8, generator=g) for _ in range(n)]


def test_tiered_prefix_cache_demotes_promotes_and_spills(tmp_path):
    c = TieredPrefixCache(PrefixCacheConfig(block_size=16, max_gpu_blocks=2, max_ram_blocks=1, disk_path=str(tmp_path)))
    toks = list(range(70))                      # 4 full blocks + 6 tokens
    kv = _kv_blocks(4)
    assert c.store_prefix(toks, kv) == 4 and len(c) == 4
    u = c.memory_usage()
    assert (u["gpu_blocks"], u["ram_blocks"], u["disk_blocks"]) == (2, 1, 1)
    m = c.match_prefix(toks)
    assert m.num_tokens == 64 and m.tiers[0] is StorageTier.DISK and m.tiers[-1] is StorageTier.GPU
    got = c.get_blocks(m.block_hashes)
    for a, b in zip(got, kv):
        assert torch.equal(a, b)                # contents survive RAM and disk
    assert c.metrics.promotions >= 2 and c.metrics.disk_reads >= 1      # small tiers: promoting one block spills others
    # acquired blocks cannot be evicted: all four now sit on the "GPU" tier although it is over budget
    assert all(c.blocks[h].tier is StorageTier.GPU for h in m.block_hashes)
    c.release_blocks(m.block_hashes)
    assert c.match_prefix(list(range(16)) + [999] * 16).num_tokens == 16
    assert c.store_prefix(toks, kv) == 0 and 0 < c.metrics.hit_rate() <= 1
    c.clear()
    assert len(c) == 0 and not list(tmp_path.iterdir())


def test_radix_cache_partial_match_and_drop():
    c = RadixPrefixCache(PrefixCacheConfig(block_size=4, max_gpu_blocks=8, max_ram_blocks=0))
    c.store_prefix([1, 2, 3, 4, 5, 6, 7, 8], [torch.zeros(1), torch.ones(1)])
    c.store_prefix([1, 2, 3, 4, 9, 9, 9, 9], [torch.zeros(1), torch.full((1,), 2.0)])
    m = c.match_prefix([1, 2, 3, 4, 5, 6, 0, 0, 1])
    assert m.num_tokens == 4 and m.partial_tokens == 2 and len(c) == 3
    n, blocks = c.extend_from_cache([1, 2, 3, 4, 9, 9, 9, 9, 5])
    assert n == 8 and float(blocks[1]) == 2.0
    small = RadixPrefixCache(PrefixCacheConfig(block_size=4, max_gpu_blocks=1, max_ram_blocks=0))
    small.store_prefix([1, 2, 3, 4, 5, 6, 7, 8], [torch.zeros(1), torch.ones(1)])
    assert len(small) == 1 and small.match_prefix([1, 2, 3, 4, 5, 6, 7, 8]).num_tokens == 0     # first block dropped: chain broken


def test_request_batcher_windows():
    from metal_marlin_b200.serving.batching import BatchConfig, RequestBatcher

    async def run():
        b = RequestBatcher(BatchConfig(max_batch_size=3, min_batch_size=2, max_wait_ms=20))
        futs = [await b.submit(i) for i in range(5)]

        async def worker():
            sizes = []
            while sum(sizes) < 5:
                batch = await b.get_batch()
                sizes.append(len(batch))
                b.complete_batch(batch, [br.request * 10 for br in batch])
            return sizes
        sizes = await asyncio.wait_for(worker(), 5)
        res = [await f for f in futs]
        return sizes, res, b
    sizes, res, b = asyncio.run(run())
    assert sizes == [3, 2] and res == [0, 10, 20, 30, 40] and b.batches_formed == 2 and b.queue_depth == 0


def test_kv_cache_sharing_copy_on_write():
    from metal_marlin_b200.serving.batching import KVCacheSharing
    copies = []
    cache = PagedKVCache(32, 4, enable_prefix_cache=False, copy_fn=lambda s, d: copies.append((s, d)))
    sh = KVCacheSharing(cache)
    prompt = list(range(10))                    # 3 blocks, the last one partial
    sh.create_region("a", prompt)
    free_before = cache.alloc.num_free
    assert sh.attach("b", prompt) is not None and sh.attach("c", [1, 2, 3]) is None
    assert cache.alloc.num_free == free_before and cache.table.block_table("a") == cache.table.block_table("b")
    sh.append("b", 1)                           # writes into the shared partial block -> copied first
    assert len(copies) == 1 and cache.table.block_table("a")[-1] != cache.table.block_table("b")[-1]
    assert cache.table.block_table("a")[:2] == cache.table.block_table("b")[:2]
    st = sh.stats()
    assert st["attached"] == 1 and st["tokens_saved"] == 10 and st["members"] == 2
    sh.release("a")
    assert sh.regions[sh.prompt_key(prompt)].owner == "b"
    sh.release("b")
    assert not sh.regions and cache.alloc.num_allocated == 0


def test_wandb_shim_falls_back_to_jsonl(tmp_path, monkeypatch):
    from metal_marlin_b200.profiling.wandb_helper import WandbHelper
    monkeypatch.setenv("WANDB_MODE", "disabled")
    w = WandbHelper(str(tmp_path))
    w.init(project="p", name="n", config={"a": 1})
    w.log({"loss": torch.tensor(0.5), "tok_s": 3.0})
    w.log({"loss": 0.25}, step=7)
    w.finish()
    rows = [json.loads(l) for l in open(w.path)]
    assert w.backend == "none" and rows[0]["_event"] == "init" and rows[1]["loss"] == 0.5 and rows[2]["_step"] == 7 and rows[-1]["steps"] == 7


def test_benchmark_report_from_bench_lines(tmp_path):
    from metal_marlin_b200.profiling.benchmark_report import aggregate_results, generate_results_file
    ours = {"metric": "decode_tok_s", "value": 300.0, "unit": "tok/s", "n_gpus": 1, "ms_per_step": 3.3, "vs_baseline": 8.5, "impl": "ours",
            "config": {"model": "glm-4.7-flash (random)", "global_batch": 1, "seq_len": 4096}, "e2e": {"value": 295.0, "unit": "tok/s"},
            "ttft_ms_p50": 210.0, "extra": {"bs32_tok_s": 1900.0, "bs32_ms_per_step": 16.8}}
    eager = dict(ours, value=7.0, impl="eager", ms_per_step=140.0, e2e={"value": 7.0, "unit": "tok/s"}, extra={})
    (tmp_path / "a.log").write_text("noise\n" + json.dumps(ours) + "\n")
    (tmp_path / "b.log").write_text(json.dumps(eager) + "\n")
    (tmp_path / "k.json").write_text(json.dumps({"batch": 1, "ctx": 4096, "results": {"q_b_gemv": {"us": 4.0, "GBps": 500}}}))
    df = aggregate_results(tmp_path)
    assert len(df) == 8 and set(df["impl"]) == {"ours", "eager"}
    md = generate_results_file(tmp_path).read_text()
    assert "glm-4.7-flash" in md and "42.86 x" in md and "q_b_gemv" in md


def test_nemo_conversion_splits_fused_tensors(tmp_path):
    from metal_marlin_b200.converters import nemo
    Hq, Hk, D, hid, inter = 4, 2, 8, 32, 48
    q, k, v = torch.randn(Hq * D, hid), torch.randn(Hk * D, hid), torch.randn(Hk * D, hid)
    g = Hq // Hk
    fused = torch.cat([torch.cat([q.view(Hk, g * D, hid)[i], k.view(Hk, D, hid)[i], v.view(Hk, D, hid)[i]]) for i in range(Hk)])
    gate, up = torch.randn(inter, hid), torch.randn(inter, hid)
    sd = {"model.embedding.word_embeddings.weight": torch.randn(100, hid), "model.decoder.layers.0.self_attention.linear_qkv.weight": fused,
          "model.decoder.layers.0.self_attention.linear_qkv.layer_norm_weight": torch.ones(hid),
          "model.decoder.layers.0.self_attention.linear_proj.weight": torch.randn(hid, Hq * D),
          "model.decoder.layers.0.mlp.linear_fc1.weight": torch.cat([gate, up]), "model.decoder.layers.0.mlp.linear_fc1.layer_norm_weight": torch.ones(hid),
          "model.decoder.layers.0.mlp.linear_fc2.weight": torch.randn(hid, inter), "model.decoder.final_layernorm.weight": torch.ones(hid),
          "model.output_layer.weight": torch.randn(100, hid), "model.decoder.layers.0.self_attention.linear_qkv._extra_state": torch.zeros(1)}
    cfg = {"num_attention_heads": Hq, "num_query_groups": Hk, "hidden_size": hid, "num_layers": 1, "ffn_hidden_size": inter, "kv_channels": D}
    path = tmp_path / "m.nemo"
    with tarfile.open(path, "w") as tf:
        for name, payload in (("model_config.yaml", yaml.safe_dump(cfg).encode()),):
            ti = tarfile.TarInfo(name); ti.size = len(payload); tf.addfile(ti, io.BytesIO(payload))
        buf = io.BytesIO(); torch.save(sd, buf); payload = buf.getvalue()
        ti = tarfile.TarInfo("model_weights.ckpt"); ti.size = len(payload); tf.addfile(ti, io.BytesIO(payload))
    out, hf = nemo.load_nemo(str(path))
    L = "model.layers.0."
    assert torch.equal(out[L + "self_attn.q_proj.weight"], q) and torch.equal(out[L + "self_attn.k_proj.weight"], k)
    assert torch.equal(out[L + "self_attn.v_proj.weight"], v) and torch.equal(out[L + "mlp.gate_proj.weight"], gate)
    assert torch.equal(out[L + "mlp.up_proj.weight"], up) and "lm_head.weight" in out and "model.norm.weight" in out
    assert hf["num_key_value_heads"] == Hk and hf["head_dim"] == D and not any("_extra_state" in k for k in out)


def test_gguf_extra_block_types_shapes_and_codebook():
    from metal_marlin_b200.converters import gguf as G
    rng = np.random.default_rng(1)
    for t in (G.Q2_K, G.Q5_K, G.IQ4_NL, G.IQ4_XS):
        n, nbytes = G.BLOCK[t]
        raw = rng.integers(0, 256, 2 * nbytes, dtype=np.uint8)
        out = G.dequantize_blocks(raw, t, 2 * n)
        assert out.shape == (2 * n,) and out.dtype == np.float32
    blk = np.zeros(18, np.uint8)
    blk[:2] = np.frombuffer(np.float16(2.0).tobytes(), dtype=np.uint8)
    blk[2:] = 0xF0                                   # low nibble code 0 (-127), high nibble code 15 (113)
    y = G.dequant_iq4_nl(blk)
    assert np.all(y[:16] == -254.0) and np.all(y[16:] == 226.0)


def test_early_exit_stops_when_confident_and_matches_full_depth_otherwise():
    from metal_marlin_b200.inference.early_exit import EarlyExitModel
    from metal_marlin_b200.models.mmfp4_causal_lm import MMFP4ForCausalLM
    from metal_marlin_b200.models.transformer import BatchMeta
    lm = MMFP4ForCausalLM.from_config("tiny-llama", device="cpu", seed=1)
    ids = torch.tensor([3, 7, 11, 200, 5])
    T = ids.numel()

    def meta():
        return BatchMeta(positions=torch.arange(T, dtype=torch.int32), slots=torch.arange(T), block_tables=torch.arange(2, dtype=torch.int32).view(1, 2),
                         ctx_lens=torch.tensor([T], dtype=torch.int32), decode=False, cu_seqlens=[0, T], ctx_lens_host=[T])
    full = lm.model.forward(ids, lm.new_cache(2, 16), meta(), last_only=True)
    never = EarlyExitModel(lm.model, exit_threshold=2.0)(ids, lm.new_cache(2, 16), meta(), rows=torch.tensor([T - 1]))
    assert never.exit_layer == len(lm.model.layers) - 1 and torch.allclose(never.logits, full, atol=1e-4)
    ee = EarlyExitModel(lm.model, exit_threshold=0.0)
    always = ee(ids, lm.new_cache(2, 16), meta(), rows=torch.tensor([T - 1]))
    assert always.exit_layer == 0 and always.logits.shape == full.shape and ee.average_exit_layer() == 0.0


def test_arena_compaction_moves_live_blocks_and_keeps_pinned_ones():
    from metal_marlin_b200.memory.arena import Arena
    a = Arena(4096, alignment=256)
    t = [a.alloc((256,), torch.uint8, tag=str(i)) for i in range(8)]            # eight 256-byte blocks
    for i, x in enumerate(t):
        x.fill_(i + 1)
    a.pin(t[5])
    for i in (0, 2, 4, 6):
        a.free(t[i])
    assert a.stats()["largest_free"] == 2048 and a.stats()["fragmentation"] > 0      # four holes + the tail
    remap = a.compact()
    # block 1 -> 0, block 3 -> 256; block 5 is pinned at 1280 and stays; block 7 follows it at 1536 (it moves from 1792)
    assert remap == {256: 0, 768: 256, 1792: 1536}
    for old, val in ((256, 2), (768, 4), (1792, 8)):
        assert torch.all(a.view_at(remap[old], (256,), torch.uint8) == val)
    assert torch.all(a.view_at(1280, (256,), torch.uint8) == 6)
    big = a.alloc((2304,), torch.uint8)                                          # the tail is one hole now
    assert a.offset_of(big) == 1792


def test_stream_pool_event_pool_and_discovery_degrade_without_cuda():
    from metal_marlin_b200.memory import streams
    pool = streams.StreamPool()
    try:
        pool.get("bogus")
        assert False
    except ValueError:
        pass
    ev = streams.EventPool().record()
    if not torch.cuda.is_available():
        assert pool.get("copy") is None and ev.wait(0.01) and streams.discover_devices() == []
    devs = [streams.DeviceInfo(i, "B200", 148, 180 << 30, (10, 0), [j for j in range(4) if j != i], 18) for i in range(4)]
    assert streams.multicast_plausible(devs)
    devs[0].peers.pop()
    assert not streams.multicast_plausible(devs)

    class FakeNvml:
        def nvmlDeviceGetHandleByIndex(self, i):
            return i

        def nvmlDeviceGetNvLinkState(self, h, link):
            if link >= 6:
                raise RuntimeError("no such link")
            return link % 2 == 0
    assert streams._nvml_links(0, FakeNvml()) == 3


def test_psd_helpers():
    from metal_marlin_b200.quant import psd
    torch.manual_seed(0)
    X = torch.randn(64, 16)
    H = X.t() @ X
    assert psd.min_eigenvalue(H) > 0 and psd.gershgorin_is_psd(torch.eye(4) * 3 + 0.5)
    bad = H - 50 * torch.eye(16)
    assert psd.min_eigenvalue(bad) < 0 and not psd.gershgorin_is_psd(bad)
    P = psd.project_psd(bad, eps=1e-3)
    assert psd.min_eigenvalue(P) > 0 and torch.allclose(P, P.t(), atol=1e-5)
    Hd, L, lam = psd.damp_until_cholesky(H)
    assert lam > 0 and torch.allclose(L @ L.t(), Hd, atol=1e-3)
    sing = torch.zeros(8, 8)
    sing[0, 0] = 1.0
    Hd, L, lam = psd.damp_until_cholesky(sing)
    assert torch.isfinite(L).all()
