"""Mixed-bit MoE path selector with feedback and A/B runs, routing cache, expert activation-buffer pool, and the random
trellis factories (reference ``tests/test_kernel_selection_mixed.py``, ``test_trellis_dispatcher_routing_cache.py``,
``trellis/testing.py`` users)."""
import random

import pytest
import torch

from metal_marlin_b200 import ops
from metal_marlin_b200.trellis import (ExpertMemoryPool, ExpertSelectionCache, MixedKernelSelector, create_mini_config, create_mini_model,
                                       create_mock_dense_mlp, create_mock_moe_mlp, create_mock_trellis_linear, get_kernel_for_batch_size,
                                       select_intelligent_kernel)
from metal_marlin_b200.trellis.kernel_selection import (FAST_2BIT_FAMILY, GROUPED_GEMM, GROUPED_GEMV, MIXED_BPW_FAMILY, SLOT_GEMV, UNIFORM_FAMILY,
                                                        bit_family)


class _Rng:
    def __init__(self, pick):
        self.pick = pick

    def random(self):
        return 0.0

    def choice(self, xs):
        return self.pick if self.pick in xs else xs[0]


def test_static_rule_and_families():
    a, b = ops.MOE_GEMV_MAX_T, ops.MOE_GROUPED_GEMV_MAX_T
    assert get_kernel_for_batch_size(1) == SLOT_GEMV and get_kernel_for_batch_size(a) == SLOT_GEMV and get_kernel_for_batch_size(a + 1) == GROUPED_GEMV
    assert get_kernel_for_batch_size(b) == GROUPED_GEMV and get_kernel_for_batch_size(b + 1) == GROUPED_GEMM
    assert bit_family([4, 4]) == UNIFORM_FAMILY and bit_family([]) == UNIFORM_FAMILY and bit_family([2, 2, 2, 4]) == FAST_2BIT_FAMILY
    assert bit_family([2, 3, 4, 2]) == MIXED_BPW_FAMILY
    assert select_intelligent_kernel(1, [4, 4]) == SLOT_GEMV


def test_heuristics_overrides_and_feedback():
    s = MixedKernelSelector(history_len=10, initial_exploration_rate=0.0)
    a = ops.MOE_GEMV_MAX_T
    k, info = s.select_kernel(a + 2, [2, 2, 2, 4])
    assert k == SLOT_GEMV and info["heuristic_family"] == FAST_2BIT_FAMILY and info["baseline_kernel"] == GROUPED_GEMV and info["reason"] == "heuristic"
    k, info = s.select_kernel(a + 2, [2, 3, 4, 2])
    assert k == GROUPED_GEMV and info["heuristic_family"] == MIXED_BPW_FAMILY
    k, info = s.select_kernel(4096, [4, 4, 4, 4], gpu_memory_pressure=0.95)
    assert k == GROUPED_GEMV and info["reason"] == "memory_pressure"
    assert s.select_kernel(1, [4], gpu_memory_pressure=0.95)[1]["reason"] == "heuristic"        # the streaming paths need no workspace
    k, info = s.select_kernel(a + 2, [2, 2, 2, 4], expert_activation_pattern={"top_expert_share": 0.9})
    assert k == GROUPED_GEMV and info["reason"] == "activation_pattern_skewed"
    k, info = s.select_kernel(1, [4, 4], available_kernels={GROUPED_GEMM})
    assert k == GROUPED_GEMM and info["reason"] == "availability_fallback"
    for _ in range(5):
        s.record_timing(SLOT_GEMV, 1, 10.0)
        s.record_timing(GROUPED_GEMV, 1, 5.0)
    k, info = s.select_kernel(1, [4, 4, 4, 4], available_kernels={SLOT_GEMV, GROUPED_GEMV})
    assert k == GROUPED_GEMV and info["reason"] == "feedback_optimization"
    assert s.select_kernel(40, [4, 4])[1]["reason"] == "heuristic"                                # timings of another bucket do not apply
    st = s.get_statistics()
    assert st["total_selections"] == 8 and st["reasons"]["feedback_optimization"] == 1 and st["timings"][f"{SLOT_GEMV}@1"]["mean_ms"] == 10.0
    few = MixedKernelSelector(history_len=2)
    for ms in (1.0, 2.0, 9.0):
        few.record_timing(SLOT_GEMV, 3, ms)
    assert list(few.timings[(SLOT_GEMV, 4)].samples) == [2.0, 9.0]


def test_ab_testing_and_accuracy():
    times = {SLOT_GEMV: 4.0, GROUPED_GEMV: 2.0, GROUPED_GEMM: 10.0}
    s = MixedKernelSelector(history_len=10, initial_exploration_rate=1.0, rng=_Rng(GROUPED_GEMV))
    k, info = s.select_kernel(1, [4, 4, 4, 4], available_kernels={SLOT_GEMV, GROUPED_GEMV}, benchmark_kernel=times.__getitem__)
    assert k == GROUPED_GEMV and info["reason"] == "ab_testing_runtime" and info["ab_test"]["winner"] == GROUPED_GEMV
    assert s.get_statistics()["ab_tests_run"] == 1 and s.get_statistics()["selection_accuracy"] == 0.0
    good = MixedKernelSelector(initial_exploration_rate=1.0, rng=_Rng(GROUPED_GEMM))
    k, info = good.select_kernel(1, [4, 4], benchmark_kernel=times.__getitem__)
    assert k == SLOT_GEMV and info["ab_test"]["challenger"] == GROUPED_GEMM and good.get_statistics()["selection_accuracy"] == 1.0
    assert good.timings[(GROUPED_GEMM, 1)].mean_ms == 10.0                                       # A/B runs feed the timing history
    off = MixedKernelSelector(initial_exploration_rate=0.0, rng=random.Random(0))
    assert off.select_kernel(1, [4], benchmark_kernel=times.__getitem__)[1]["reason"] == "heuristic"


def test_selection_cache_and_memory_pool():
    c = ExpertSelectionCache(capacity=2)
    ids = torch.tensor([[0, 3], [1, 2]])
    built = []
    g = c.get_or_build(ids, lambda t: built.append(1) or {"order": t.reshape(-1).argsort()})
    assert c.get_or_build(ids.clone(), lambda t: built.append(1)) is g and built == [1] and c.hit_rate() == 0.5
    assert c.get(ids.reshape(1, 4)) is None                                                       # same ids, another shape
    c.put(torch.tensor([[5, 6]]), "a")
    c.put(torch.tensor([[7, 8]]), "b")
    assert c.get(ids) is None and c.get(torch.tensor([[7, 8]])) == "b"
    c.clear()
    assert c.hit_rate() == 0.0
    p = ExpertMemoryPool("cpu", max_buffers_per_bucket=1)
    a = p.acquire(5, 64, torch.float32)
    assert a.shape == (5, 64) and a._base.shape == (8, 64)
    p.release(a)
    b = p.acquire(7, 64, torch.float32)
    assert b._base is a._base and p.stats()["reuses"] == 1 and p.stats()["allocations"] == 1
    c2 = p.acquire(7, 64, torch.float32)
    p.release(b)
    p.release(c2)                                                                                 # the bucket keeps one
    assert p.stats()["bytes_held"] == 8 * 64 * 4 and p.acquire(9, 64, torch.float32)._base.shape == (16, 64)
    p.clear()
    assert p.stats()["bytes_held"] == 0


def test_random_trellis_factories():
    lin = create_mock_trellis_linear(128, 64, bits=3, seed=1)
    x = torch.randn(3, 128)
    assert lin(x).shape == (3, 64) and lin.bits == 3
    assert torch.equal(create_mock_trellis_linear(128, 64, bits=3, seed=1)(x), lin(x))           # seeded
    mlp = create_mock_dense_mlp(128, 256, bits=4)
    assert mlp(x).shape == (3, 128)
    moe = create_mock_moe_mlp(128, 128, num_experts=4, top_k=2, bits=(2, 3, 4), num_shared_experts=1)
    assert [e.gate.bits for e in moe.experts] == [2, 3, 4, 2] and len(moe.shared) == 1
    y = moe(x)
    assert y.shape == x.shape and torch.isfinite(y.float()).all()
    cfg = create_mini_config(num_layers=2)
    assert cfg.num_hidden_layers == 2 and cfg.is_moe
    lm = create_mini_model(cfg)
    assert torch.isfinite(lm.forward_logits([1, 2, 3]).float()).all()
    assert not create_mini_config(moe=False).is_moe
