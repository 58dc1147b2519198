"""Paged-cache bookkeeping, scheduler policies and the engine loop (CPU).  Behavioural specs taken from the
reference's tests/test_paged.py, test_cow_cache_manager.py, test_batch_scheduler.py and test_continuous_batch*.py."""
import pytest
import torch

from metal_marlin_b200.engine.engine import EngineConfig, LLMEngine
from metal_marlin_b200.engine.request import (GenerationRequest, IllegalTransition, RequestPriority, RequestStatus,
                                              RunningRequest)
from metal_marlin_b200.engine.scheduler import BatchScheduler, PreemptionPolicy, QueueFullError, SchedulerConfig
from metal_marlin_b200.engine.session import SamplingParams
from metal_marlin_b200.kv.paged import (BlockAllocator, EvictionPolicy, MultimodalBlockAllocator, OutOfBlocks, PagedKVCache,
                                        PageTable, PrefixCache)
from metal_marlin_b200.models.mmfp4_causal_lm import MMFP4ForCausalLM


# ---------------------------------------------------------------- allocator / page table
def test_allocator_refcount_and_free():
    a = BlockAllocator(4, 16)
    b0, b1 = a.allocate(), a.allocate()
    assert (b0, b1) == (0, 1) and a.num_free == 2
    a.incref(b0)
    a.free(b0)
    assert a.num_free == 2 and a.ref_count(b0) == 1
    a.free(b0)
    assert a.num_free == 3
    with pytest.raises(AssertionError):
        a.free(b0)
    a.allocate_many(3)
    with pytest.raises(OutOfBlocks):
        a.allocate()


def test_allocator_contiguous_best_fit_and_fragmentation():
    a = BlockAllocator(12, 16)
    ids = a.allocate_many(12)
    for b in (1, 2, 5, 6, 7, 8, 10):
        a.free(b)
    assert a.free_runs() == [(1, 2), (5, 4), (10, 1)]
    assert a.allocate_contiguous(2) == [1, 2]          # smallest run that fits, not the first 4-run
    assert a.allocate_contiguous(3) == [5, 6, 7]
    assert 0.0 < a.fragmentation() <= 0.5
    with pytest.raises(OutOfBlocks):
        a.allocate_contiguous(3)


def test_copy_on_write():
    a = BlockAllocator(4, 16)
    copies = []
    b = a.allocate()
    assert a.cow(b, lambda s, d: copies.append((s, d))) == b and not copies
    a.incref(b)
    nb = a.cow(b, lambda s, d: copies.append((s, d)))
    assert nb != b and copies == [(b, nb)] and a.ref_count(b) == 1 and a.cow_copies == 1


def test_page_table_append_fork_truncate():
    a = BlockAllocator(8, 4)
    pt = PageTable(a)
    pt.add_sequence("a", 6)
    assert len(pt.block_table("a")) == 2
    assert pt.slot_mapping("a", 0, 6) == [0, 1, 2, 3, 4, 5]
    pt.fork("a", "b")
    assert a.ref_count(pt.block_table("a")[1]) == 2
    slots = pt.append_tokens("b", 1)                      # writes into the shared half-full block -> COW
    assert pt.block_table("b")[1] != pt.block_table("a")[1] and slots == [pt.block_table("b")[1] * 4 + 2]
    pt.append_tokens("a", 3)
    assert pt.num_tokens("a") == 9 and len(pt.block_table("a")) == 3
    pt.truncate("a", 5)
    assert pt.num_tokens("a") == 5 and len(pt.block_table("a")) == 2
    pt.remove("a"), pt.remove("b")
    assert a.num_free == 8


def test_prefix_cache_match_insert_evict():
    a = BlockAllocator(16, 4)
    pc = PrefixCache(a, max_blocks=3, policy=EvictionPolicy.LRU)
    toks = list(range(10))
    blocks = a.allocate_many(3)
    assert pc.insert(toks, blocks) == 2                   # only full blocks are cached
    assert pc.match(toks) == blocks[:2] and a.ref_count(blocks[0]) == 3
    assert pc.match([0, 1, 2, 3, 99, 5, 6, 7]) == blocks[:1]
    assert pc.match([9, 9, 9, 9]) == []
    pc.insert(list(range(100, 108)), a.allocate_many(2))  # exceeds max_blocks -> LRU eviction
    assert len(pc.table) == 3 and pc.evictions == 1


def test_paged_cache_admit_uses_prefix_and_never_the_last_block():
    kv = PagedKVCache(16, 4)
    toks = list(range(12))
    assert kv.admit("a", toks) == 0
    kv.publish("a", toks)
    assert kv.admit("b", toks) == 8                       # 12 tokens = 3 full blocks, last one recomputed
    assert kv.table.block_table("b")[:2] == kv.table.block_table("a")[:2]
    kv.release("a"), kv.release("b")
    assert kv.alloc.num_free == 16 - len(kv.prefix.table)


def test_multimodal_allocator_shares_image_blocks():
    a = MultimodalBlockAllocator(16, 4, vision_fraction=0.5)
    x = a.allocate_image("img", 10)
    y = a.allocate_image("img", 10)
    assert x == y and a.ref_count(x[0]) == 2
    with pytest.raises(OutOfBlocks):
        a.allocate_image("big", 40)
    a.release_image("img"), a.release_image("img")
    assert a.num_free == 16


# ---------------------------------------------------------------- request FSM
def test_request_state_machine():
    rr = RunningRequest(GenerationRequest([1, 2, 3], 4))
    with pytest.raises(IllegalTransition):
        rr.transition(RequestStatus.RUNNING)
    rr.transition(RequestStatus.PREFILLING)
    rr.transition(RequestStatus.RUNNING)
    rr.append_token(7)
    assert rr.ttft is not None and rr.should_stop() is None
    rr.transition(RequestStatus.PREEMPTED)
    assert rr.prefill_target == 3
    rr.transition(RequestStatus.PREFILLING)
    rr.transition(RequestStatus.FINISHED)
    assert rr.done.is_set()
    with pytest.raises(IllegalTransition):
        rr.transition(RequestStatus.RUNNING)


# ---------------------------------------------------------------- scheduler
def _sched(blocks=64, **kw):
    cfg = SchedulerConfig(block_size=4, **kw)
    return BatchScheduler(cfg, PagedKVCache(blocks, 4, enable_prefix_cache=False))


def _drive(s, out, tok=5):
    sampled = {}
    for ch in out.prefill:
        if ch.start + ch.length >= ch.request.prefill_target and not ch.request.output_ids:
            sampled[ch.request.id] = tok
    for rr in out.decode:
        sampled[rr.id] = tok
    return s.step(out, sampled)


def test_chunked_prefill_then_decode_and_budgets():
    s = _sched(max_num_batched_tokens=16, max_prefill_tokens=8, max_chunk=6)
    a = s.add_request(GenerationRequest(list(range(10)), 3))
    o = s.schedule()
    assert [(c.start, c.length) for c in o.prefill] == [(0, 6)] and not o.decode
    _drive(s, o)
    o = s.schedule()
    assert [(c.start, c.length) for c in o.prefill] == [(6, 4)]
    _drive(s, o)
    assert a.status is RequestStatus.RUNNING and a.output_ids == [5]
    b = s.add_request(GenerationRequest(list(range(20)), 2))
    o = s.schedule()
    assert o.decode == [a] and o.prefill[0].request is b and o.prefill[0].length == 6      # decode first, prefill after
    assert o.num_tokens <= 16


def test_priority_order_and_starvation_promotion():
    s = _sched(max_num_seqs=1, starvation_s=0.0)
    lo = s.add_request(GenerationRequest([1, 2], 1, priority=RequestPriority.LOW))
    hi = s.add_request(GenerationRequest([3, 4], 1, priority=RequestPriority.HIGH))
    o = s.schedule()
    assert o.prefill[0].request is hi
    assert lo.effective_priority > int(RequestPriority.LOW)       # promoted while it waited


def test_preemption_by_recompute_when_blocks_run_out():
    s = _sched(blocks=4, preemption_policy=PreemptionPolicy.LOWEST_PRIORITY)
    a = s.add_request(GenerationRequest(list(range(7)), 8, priority=RequestPriority.HIGH))
    b = s.add_request(GenerationRequest(list(range(7)), 8, priority=RequestPriority.LOW))
    _drive(s, s.schedule())
    assert a.status is RequestStatus.RUNNING and b.status is RequestStatus.RUNNING and s.cache.alloc.num_free == 0
    _drive(s, s.schedule())                              # both decode into their half-empty second block
    o = s.schedule()                                     # now each needs a third block: the low-priority one is evicted
    assert b in o.preempted and b.status is RequestStatus.PREEMPTED and b.prefill_progress == 0
    assert a in o.decode and s.num_preemptions == 1
    _drive(s, o)
    while a.status is not RequestStatus.FINISHED:
        _drive(s, s.schedule())
    while b.status is not RequestStatus.FINISHED:
        _drive(s, s.schedule())
    assert len(b.output_ids) == 8 and b.num_preemptions >= 1
    assert s.cache.alloc.num_free == 4


def test_queue_full_and_abort():
    s = _sched(max_waiting=1)
    a = s.add_request(GenerationRequest([1], 1))
    with pytest.raises(QueueFullError):
        s.add_request(GenerationRequest([1], 1))
    assert s.abort(a.id) and a.status is RequestStatus.ABORTED and not s.has_work()


# ---------------------------------------------------------------- engine
def test_engine_matches_plain_generate_and_reuses_prefixes():
    lm = MMFP4ForCausalLM.from_config("tiny-llama", device="cpu", seed=0)
    prompts = [list(range(1, 40)), list(range(1, 40)) + [77, 78], [9, 8, 7]]
    want = [lm.generate([p], max_new_tokens=6)[0] for p in prompts]
    eng = LLMEngine(lm.model, EngineConfig(num_kv_blocks=64, block_size=16, max_model_len=128, max_chunk=16,
                                           max_prefill_tokens=32, use_cuda_graphs=False))
    got = eng.generate(prompts, max_new_tokens=6)
    assert got == want
    assert eng.cache.alloc.num_free == 64 - len(eng.cache.prefix.table)
    got2 = eng.generate([prompts[0]], max_new_tokens=6)       # second pass hits the prefix cache
    assert got2[0] == want[0] and eng.cache.prefix.hits >= 1


def test_engine_background_thread_streams_tokens():
    lm = MMFP4ForCausalLM.from_config("tiny-llama", device="cpu", seed=0)
    eng = LLMEngine(lm.model, EngineConfig(num_kv_blocks=32, max_model_len=64, use_cuda_graphs=False))
    eng.start()
    seen = []
    rr = eng.add_request(GenerationRequest([1, 2, 3], 5, on_token=lambda rid, t: seen.append(t)))
    assert rr.done.wait(30)
    eng.stop()
    assert rr.status is RequestStatus.FINISHED and seen == rr.output_ids and len(seen) == 5


def test_engine_survives_preemption_with_identical_output():
    lm = MMFP4ForCausalLM.from_config("tiny-llama", device="cpu", seed=0)
    prompts = [list(range(1, 30)), list(range(40, 70))]
    want = [lm.generate([p], max_new_tokens=10)[0] for p in prompts]
    eng = LLMEngine(lm.model, EngineConfig(num_kv_blocks=5, block_size=16, max_model_len=64, enable_prefix_cache=False,
                                           use_cuda_graphs=False))
    got = eng.generate(prompts, max_new_tokens=10)
    assert got == want and eng.scheduler.num_preemptions >= 1


def test_engine_fails_requests_when_the_device_status_word_is_set():
    """A bounded in-kernel wait that ran out leaves a code in the device status word; the engine reads the word back with
    the sampled ids, fails the in-flight requests instead of returning their tokens, and clears the word."""
    from metal_marlin_b200 import ops
    from metal_marlin_b200.parallel.health import DeviceWaitExpired, PeerFailure
    lm = MMFP4ForCausalLM.from_config("tiny-llama", device="cpu", seed=0)
    eng = LLMEngine(lm.model, EngineConfig(num_kv_blocks=32, max_model_len=64, use_cuda_graphs=False))
    st = ops.gemm_status(lm.device)
    eng.add_request(GenerationRequest([1, 2, 3], 4))
    st[0] = 101                                   # as if the wait on tensor-parallel source 1 had expired
    with pytest.raises(PeerFailure) as e:
        eng.step()                                # prompt pass
    assert e.value.ranks == [1] and int(st[0]) == 0
    eng.step()                                    # the word was cleared: the next pass runs
    st[0] = 200                                   # paged-decode barrier: a local wait, no rank named
    with pytest.raises(DeviceWaitExpired):
        eng.step()                                # decode pass
    assert int(st[0]) == 0
    # expert-parallel receive-buffer overflow (120): fails the step unless the model asked for token dropping
    from metal_marlin_b200.parallel.health import ExpertCapacityOverflow
    st[0] = 120
    with pytest.raises(ExpertCapacityOverflow):
        eng.step()

    class _EP:
        capacity_policy, overflow_steps, mode, pass_tokens = "drop", 0, "nccl", 0
    lm.model.ep = _EP()
    try:
        eng3 = LLMEngine(lm.model, EngineConfig(num_kv_blocks=32, max_model_len=64, use_cuda_graphs=False))
        eng3.cache, eng3.kv = eng.cache, eng.kv
        st[0] = 120
        eng3._check_device_status()               # tolerated, counted, cleared
        assert lm.model.ep.overflow_steps == 1 and int(st[0]) == 0
    finally:
        lm.model.ep = None
    # background loop: the in-flight request ends FAILED with the reason, the loop keeps serving
    eng2 = LLMEngine(lm.model, EngineConfig(num_kv_blocks=32, max_model_len=64, use_cuda_graphs=False))
    st[0] = 3
    eng2.start()
    bad = eng2.add_request(GenerationRequest([4, 5, 6], 4))
    assert bad.done.wait(30) and bad.status is RequestStatus.FAILED and "status 3" in bad.error
    good = eng2.add_request(GenerationRequest([4, 5, 6], 4))
    assert good.done.wait(30) and good.status is RequestStatus.FINISHED
    eng2.stop()


def test_engine_applies_repetition_penalty_per_request():
    """The penalty of each request reaches the sampler together with that request's recent tokens (prompt tail and
    generated ids): with a very strong penalty nothing already seen is produced again."""
    lm = MMFP4ForCausalLM.from_config("tiny-llama", device="cpu", seed=0)
    eng = LLMEngine(lm.model, EngineConfig(num_kv_blocks=32, max_model_len=128, use_cuda_graphs=False))
    prompt = list(range(10, 30))
    plain = eng.add_request(GenerationRequest(list(prompt), 12))
    pen = eng.add_request(GenerationRequest(list(prompt), 12, SamplingParams(repetition_penalty=1e4)))
    eng.run_until_done()
    assert len(set(pen.output_ids)) == len(pen.output_ids) and not set(pen.output_ids) & set(prompt)
    assert plain.output_ids != pen.output_ids or len(set(plain.output_ids)) == len(plain.output_ids)


def test_preemption_by_swap_plans_block_moves_and_resumes_without_recompute():
    s = _sched(blocks=4, preemption_policy=PreemptionPolicy.LOWEST_PRIORITY, preemption_mode="swap", swap_space_blocks=4)
    a = s.add_request(GenerationRequest(list(range(7)), 8, priority=RequestPriority.HIGH))
    b = s.add_request(GenerationRequest(list(range(7)), 8, priority=RequestPriority.LOW))
    _drive(s, s.schedule())
    _drive(s, s.schedule())
    o = s.schedule()                                     # each needs a third block: the low-priority one goes to the host
    assert b.status is RequestStatus.SWAPPED and b in o.preempted and s.swapped_out == [b] and b.prefill_progress == 7
    (rr, dev_blocks, host_blocks), = o.swap_out
    assert rr is b and len(dev_blocks) == len(host_blocks) == 2 and b.swap_tokens == len(b.all_ids) - 1 == 8
    assert a in o.decode and s.num_swaps == 1 and len(s._host_free) == 2
    _drive(s, o)
    c = s.add_request(GenerationRequest(list(range(3)), 2, priority=RequestPriority.REALTIME))
    while a.status is not RequestStatus.FINISHED:
        o = s.schedule()
        assert not o.swap_in and c.status is RequestStatus.WAITING       # nothing new is admitted past a swapped sequence
        _drive(s, o)
    o = s.schedule()
    (rr, host_back, dev_new), = o.swap_in
    assert rr is b and host_back == host_blocks and len(dev_new) == 2 and b.status is RequestStatus.RUNNING
    assert s.cache.table.num_tokens(b.id) == 8 and len(s._host_free) == 4
    _drive(s, o)
    while s.has_work():
        _drive(s, s.schedule())
    assert len(b.output_ids) == 8 and c.status is RequestStatus.FINISHED and s.cache.alloc.num_free == 4
    # a swapped request can be aborted: its host blocks return
    s2 = _sched(blocks=4, preemption_mode="swap", swap_space_blocks=2)
    x = s2.add_request(GenerationRequest(list(range(7)), 8, priority=RequestPriority.HIGH))
    y = s2.add_request(GenerationRequest(list(range(7)), 8, priority=RequestPriority.LOW))
    for _ in range(3):
        _drive(s2, s2.schedule())
    assert y.status is RequestStatus.SWAPPED and s2.abort(y.id) and len(s2._host_free) == 2 and not s2.swapped_out
    # without host room the victim is recomputed as before
    s3 = _sched(blocks=4, preemption_mode="swap", swap_space_blocks=1)
    s3.add_request(GenerationRequest(list(range(7)), 8, priority=RequestPriority.HIGH))
    z = s3.add_request(GenerationRequest(list(range(7)), 8, priority=RequestPriority.LOW))
    for _ in range(3):
        _drive(s3, s3.schedule())
    assert z.status is RequestStatus.PREEMPTED and z.prefill_progress == 0


@pytest.mark.parametrize("kv_dtype", ["bf16", "fp8"])
def test_engine_swap_preemption_keeps_the_output(kv_dtype):
    lm = MMFP4ForCausalLM.from_config("tiny-llama", device="cpu", seed=0)
    prompts = [list(range(1, 30)), list(range(40, 70))]
    base = LLMEngine(lm.model, EngineConfig(num_kv_blocks=16, block_size=16, max_model_len=64, enable_prefix_cache=False,
                                            use_cuda_graphs=False, kv_cache_dtype=kv_dtype))
    want = base.generate(prompts, max_new_tokens=10)
    eng = LLMEngine(lm.model, EngineConfig(num_kv_blocks=5, block_size=16, max_model_len=64, enable_prefix_cache=False,
                                           use_cuda_graphs=False, kv_cache_dtype=kv_dtype, preemption_mode="swap"))
    got = eng.generate(prompts, max_new_tokens=10)
    st = eng.scheduler.stats()
    assert got == want and st["swaps"] >= 1 and st["swapped_out"] == 0
    assert len(eng.scheduler._host_free) == eng.swap_blocks == 5


def test_prefill_budget_follows_memory_pressure_and_recovers_from_oom():
    import torch
    from metal_marlin_b200.engine.engine import PrefillBudget
    free = {"v": 10_000_000}
    cfg = SchedulerConfig(max_prefill_tokens=1024)
    b = PrefillBudget(cfg, need_fn=lambda n: n * 1000, free_fn=lambda: free["v"], floor=128)
    assert b.before_iteration() == 1024               # 10 MB free, 1 MB needed
    free["v"] = 500_000                               # less than 1.25 x the need of 1024 and of 512 tokens, enough for 256
    assert b.before_iteration() == 512 and b.before_iteration() == 256 and cfg.max_prefill_tokens == 256
    assert b.before_iteration() == 256                # 320 tokens would need 2 x 320 kB: no room to grow
    free["v"] = 900_000                               # room for 320 (640 kB x ... ) and 400, not for 500
    assert b.before_iteration() == 320 and b.before_iteration() == 400 and b.before_iteration() == 400
    free["v"] = 10_000_000
    for _ in range(10):
        b.before_iteration()
    assert b.value == 1024 and b.shrinks == 2
    assert b.on_oom() == 512 and b.stats()["ooms"] == 1
    for _ in range(5):
        b.on_oom()
    assert b.value == 128                            # never below the floor

    # an engine whose prompt pass runs out of memory once: the chunks are planned again under half the budget
    lm = MMFP4ForCausalLM.from_config("tiny-llama", device="cpu", seed=0)
    prompts = [list(range(1, 60)), list(range(70, 100))]
    want = [lm.generate([p], max_new_tokens=6)[0] for p in prompts]
    eng = LLMEngine(lm.model, EngineConfig(num_kv_blocks=32, block_size=16, max_model_len=128, use_cuda_graphs=False,
                                           max_prefill_tokens=256, max_chunk=256, adaptive_prefill_budget=True))
    assert eng.prefill_budget.need_fn(256) > eng.prefill_budget.need_fn(128) > 0
    eng.prefill_budget.floor = 16
    real, calls = eng._exec_prefill, {"n": 0, "sizes": []}

    def flaky(a):
        calls["n"] += 1
        calls["sizes"].append(len(a["ids"]))
        if calls["n"] == 1:
            raise torch.cuda.OutOfMemoryError("simulated")
        return real(a)
    eng._exec_prefill = flaky
    got = eng.generate(prompts, max_new_tokens=6)
    assert got == want and eng.stats()["prefill_budget"]["ooms"] == 1
    assert calls["sizes"][0] == 89 and calls["sizes"][1] <= 128


def test_prefix_cache_fifo_adaptive_and_proactive_eviction():
    from metal_marlin_b200.kv.paged import BlockAllocator, EvictionPolicy, PrefixCache
    al = BlockAllocator(16, 4)
    pc = PrefixCache(al, max_blocks=8, policy=EvictionPolicy.FIFO)
    seqs = [[i] * 4 for i in range(4)]
    blocks = []
    for t in seqs:
        b = al.allocate()
        blocks.append(b)
        pc.insert(t, [b])
        al.free(b)                       # only the cache holds the block now
    for b in pc.match(seqs[0]):          # a hit does not save the oldest entry under FIFO
        al.free(b)
    assert pc.evict_one() and not pc.match(seqs[0]) and al.ref_count(blocks[0]) == 0
    assert pc.evict_batch(2) == 2 and len(pc.table) == 1
    # adaptive: with a high hit rate the never-hit entry goes although it is the most recent one
    al2 = BlockAllocator(16, 4)
    ad = PrefixCache(al2, max_blocks=8, policy=EvictionPolicy.ADAPTIVE)
    for t in seqs[:3]:
        b = al2.allocate()
        ad.insert(t, [b])
        al2.free(b)
    for _ in range(5):
        for t in seqs[:2]:
            for b in ad.match(t):
                al2.free(b)
    assert ad.evict_one() and ad.match(seqs[0]) and ad.match(seqs[1])
    assert len(ad.table) == 2
    # proactive eviction: above 75 % usage cached blocks are released until usage is back under it
    al3 = BlockAllocator(8, 4)
    pe = PrefixCache(al3, max_blocks=8)
    held = [al3.allocate() for _ in range(3)]
    for i in range(4):
        b = al3.allocate()
        pe.insert([100 + i] * 4, [b])
        al3.free(b)
    assert al3.usage() == 7 / 8 and pe.proactive_evict(0.75) == 1 and al3.usage() == 6 / 8 and len(held) == 3


def test_block_compaction_rewrites_tables_and_prefix_entries():
    moved = []
    cache = PagedKVCache(12, 4, enable_prefix_cache=True, copy_fn=lambda s, d: moved.append((s, d)))
    toks = {sid: [ord(sid) * 10 + i for i in range(8)] for sid in "abcdef"}
    for sid, t in toks.items():
        cache.admit(sid, t)
        cache.publish(sid, t)
    for sid in "ace":                         # every other sequence leaves: holes between the survivors...
        cache.release(sid)
    cache.prefix.evict_until(12)              # ...once the cache's own references to their blocks are gone too
    before = {sid: list(cache.table.block_table(sid)) for sid in "bdf"}
    assert cache.alloc.fragmentation() > 0 and not cache.alloc.needs_compaction()
    assert cache.compact() == 0               # below the thresholds nothing moves
    n = cache.compact(force=True)
    assert n == len(moved) > 0
    after = {sid: list(cache.table.block_table(sid)) for sid in "bdf"}
    remap = dict(moved)
    assert all(after[s] == [remap.get(b, b) for b in before[s]] for s in "bdf")
    used = sorted(b for bl in after.values() for b in bl)
    assert used == list(range(len(used))) and cache.alloc.fragmentation() == 0.0
    assert cache.alloc.num_free == 12 - len(used) and all(cache.alloc.ref_count(b) >= 1 for b in used)
    # allocation still works and hands out the packed free ids
    assert cache.alloc.allocate_contiguous(4) == list(range(len(used), len(used) + 4))
    al = PagedKVCache(64, 1, enable_prefix_cache=False).alloc
    ids = al.allocate_many(64)
    for b in ids[::2]:
        al.free(b)
    assert al.needs_compaction(max_runs=16)   # 32 one-block holes
