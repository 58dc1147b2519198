"""First-come-first-served scheduler: prefill strategies, insertion policies, the swapped queue, and the engine running on it."""
import pytest

from metal_marlin_b200.engine.engine import EngineConfig, LLMEngine
from metal_marlin_b200.engine.fcfs import CacheInfo, FCFSScheduler, InsertionPolicy, PrefillStrategy
from metal_marlin_b200.engine.request import GenerationRequest, RequestPriority, RequestStatus
from metal_marlin_b200.engine.scheduler import QueueFullError, SchedulerConfig
from metal_marlin_b200.kv.paged import PagedKVCache
from metal_marlin_b200.models.mmfp4_causal_lm import MMFP4ForCausalLM


def _sched(blocks=64, strategy=PrefillStrategy.FCFS, prefix=False, **kw):
    cfg = SchedulerConfig(block_size=4, **kw)
    return FCFSScheduler(cfg, PagedKVCache(blocks, 4, enable_prefix_cache=prefix), prefill_strategy=strategy)


def _drive(s, out, tok=5):
    sampled = {}
    for ch in out.prefill:
        if ch.start + ch.length >= ch.request.prefill_target and not ch.request.output_ids:
            sampled[ch.request.id] = tok
    for rr in out.decode:
        sampled[rr.id] = tok
    return s.step(out, sampled)


def _req(n, new=2, **kw):
    return GenerationRequest(list(range(1, n + 1)), new, **kw)


def test_arrival_order_ignores_priorities():
    s = _sched(max_num_seqs=1)
    lo = s.add_request(_req(3, priority=RequestPriority.LOW))
    s.add_request(_req(3, priority=RequestPriority.REALTIME))
    assert s.schedule().prefill[0].request is lo


@pytest.mark.parametrize("strategy, want", [(PrefillStrategy.FCFS, [9, 3, 6]), (PrefillStrategy.SHORTEST_FIRST, [3, 6, 9]),
                                            (PrefillStrategy.LONGEST_FIRST, [9, 6, 3])])
def test_prefill_strategies_order_admission(strategy, want):
    s = _sched(strategy=strategy, max_num_seqs=1)
    for n in (9, 3, 6):
        s.add_request(_req(n, new=1))
    order = []
    while s.has_work():
        o = s.schedule()
        order += [len(c.request.req.prompt_ids) for c in o.prefill if c.start == 0]
        _drive(s, o)
    assert order == want


def test_insertion_policies_and_stats():
    s = _sched(max_waiting=4)
    a = s.add_request(_req(2))
    assert s.insert_batch([_req(3), _req(4)], InsertionPolicy.ENQUEUE) == 2
    assert [len(r.req.prompt_ids) for r in s.waiting] == [2, 3, 4]
    assert s.insert_batch([_req(5), _req(6)], InsertionPolicy.DROP_IF_FULL) == 0          # two do not fit: none is queued
    assert s.insert_batch_front([_req(7), _req(8)]) == 1                                  # one fits; the other is counted as dropped
    assert [len(r.req.prompt_ids) for r in s.waiting] == [7, 2, 3, 4]
    assert s.insertion_stats() == {"total_inserted": 4, "total_dropped": 3, "batch_insertions": 3}
    assert s.queue_utilization() == 1.0
    with pytest.raises(QueueFullError):
        s.add_request_front(_req(1))
    assert s.clear_waiting() == 4 and a.status is RequestStatus.ABORTED and not s.has_work()
    s.reset_insertion_stats()
    front = s.add_request(_req(2))
    first = s.add_request_front(_req(9))
    assert s.schedule().prefill[0].request is first and front.status is RequestStatus.PREFILLING
    assert s.insertion_stats()["total_inserted"] == 2


def test_merge_keeps_batch_order_at_the_front():
    s = _sched()
    s.add_request(_req(2))
    s.insert_batch([_req(5), _req(6), _req(7)], "merge")
    assert [len(r.req.prompt_ids) for r in s.waiting] == [5, 6, 7, 2]


def test_preempted_sequences_wait_in_the_swapped_queue_and_come_back_first():
    s = _sched(blocks=4)
    a = s.add_request(_req(7, new=8))
    b = s.add_request(_req(7, new=8))
    _drive(s, s.schedule())
    _drive(s, s.schedule())
    o = s.schedule()                                    # a third block each: the one with the most tokens is evicted (a tie: the first)
    assert len(o.preempted) == 1 and s.num_swapped == 1 and s.num_waiting == 0
    victim = o.preempted[0]
    late = s.add_request(_req(2, new=1))
    _drive(s, o)
    seen_victim_before_late = None
    while s.has_work():
        o = s.schedule()
        for c in o.prefill:
            if c.start == 0 and seen_victim_before_late is None and c.request in (victim, late):
                seen_victim_before_late = c.request is victim
        _drive(s, o)
    assert seen_victim_before_late is True
    assert len(a.output_ids) == 8 and len(b.output_ids) == 8 and late.status is RequestStatus.FINISHED
    assert s.cache.alloc.num_free == 4
    assert {r.id for r in s.free_finished()} == {a.id, b.id, late.id} and not s.requests


def test_cache_info_reports_prefix_reuse():
    s = _sched(prefix=True)
    a = s.add_request(_req(10, new=1))
    assert s.get_cache_info(a.id) is None               # not admitted yet
    while s.has_work():
        _drive(s, s.schedule())
    b = s.add_request(_req(10, new=1))
    s.schedule()
    info = s.get_cache_info(b.id)
    assert isinstance(info, CacheInfo) and info.cache_hit and info.cached_tokens == 8 and info.uncached_tokens == 2
    assert info.cached_blocks == 2 and info.total_tokens == 10
    assert s.stats()["prefill_strategy"] == "fcfs"


@pytest.mark.parametrize("policy", ["fcfs", "shortest_first"])
def test_engine_runs_on_the_fcfs_scheduler(policy):
    lm = MMFP4ForCausalLM.from_config("tiny-llama", device="cpu", seed=0)
    prompts = [list(range(1, 30)), [9, 8, 7], list(range(40, 60))]
    want = [lm.generate([p], max_new_tokens=5)[0] for p in prompts]
    eng = LLMEngine(lm.model, EngineConfig(num_kv_blocks=32, block_size=16, max_model_len=64, use_cuda_graphs=False,
                                           scheduler_policy=policy))
    assert isinstance(eng.scheduler, FCFSScheduler)
    assert eng.generate(prompts, max_new_tokens=5) == want
