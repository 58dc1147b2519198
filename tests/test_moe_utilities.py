"""MoE utilities: capacity analysis and overflow policies, dynamic capacity, load tracking / balancing loss / gate entropy, and
the predictive expert prefetcher.  Reference: tests/test_capacity.py, tests/test_moe_prefetch.py, tests/test_load_balancing.py."""
import time

import pytest
import torch

from metal_marlin_b200.moe import (CapacityAnalyzer, DynamicCapacity, DynamicCapacityConfig, ExpertLoadTracker, ExpertPrefetcher,
                                   LoadBalancingConfig, OverflowPolicy, PrefetchConfig, PrefetchStrategy, analyze_overflow_rate,
                                   apply_overflow_policy, auto_tune_capacity, compute_expert_capacity, count_expert_assignments,
                                   gate_entropy, load_balance_loss)
from metal_marlin_b200.parallel.health import ExpertCapacityOverflow


def _skewed(T=64, E=8, k=2, seed=0):
    g = torch.Generator().manual_seed(seed)
    p = torch.softmax(torch.randn(T, E, generator=g) + torch.tensor([3.0, 1.5] + [0.0] * (E - 2)), -1)
    w, ids = torch.topk(p, k, -1)
    return p, ids.to(torch.int32), w


def test_capacity_math_and_analyzer():
    assert compute_expert_capacity(64, 8, 2, 1.25) == 20 and compute_expert_capacity(3, 64, 4, 1.0, min_capacity=4) == 4
    p, ids, w = _skewed()
    c = count_expert_assignments(ids, 8)
    assert int(c.sum()) == 128 and int(c[0]) > 40
    an = CapacityAnalyzer(8, 2, 1.25)
    info = an.record_batch(ids)
    assert info.capacity == 20 and info.dropped == int((c - 20).clamp_min(0).sum()) and 0 in info.overflow_experts
    assert 0 < info.drop_rate < 1 and 0 < info.utilization <= 1
    st = an.get_stats()
    assert st.batches == 1 and st.overflow_rate == 1.0 and st.top_overflow_experts(1)[0][0] == 0 and st.peak_load == int(c.max())
    batches = [_skewed(seed=s)[1] for s in range(6)]
    rates = analyze_overflow_rate(batches, 8, 2, (1.0, 2.0, 4.0))
    assert rates[1.0]["drop_rate"] > rates[2.0]["drop_rate"] >= rates[4.0]["drop_rate"]
    f = auto_tune_capacity(batches, 8, 2, target_drop_rate=0.02)
    assert analyze_overflow_rate(batches, 8, 2, (f,))[f]["drop_rate"] <= 0.02 < analyze_overflow_rate(batches, 8, 2, (f - 0.3,))[f - 0.3]["drop_rate"]


def test_overflow_policies():
    p, ids, w = _skewed()
    cap = 20
    d_ids, d_w, over = apply_overflow_policy(ids, w, 8, cap, OverflowPolicy.DROP)
    assert over > 0 and int((d_ids == -1).sum()) == over and int(count_expert_assignments(d_ids, 8).max()) <= cap
    assert torch.all(d_w[d_ids == -1] == 0)
    r_ids, r_w, _ = apply_overflow_policy(ids, w, 8, cap, "renorm")
    some = (r_ids != -1).any(-1)
    torch.testing.assert_close(r_w.sum(-1)[some], w.sum(-1)[some])
    m_ids, m_w, over2 = apply_overflow_policy(ids, w, 8, cap, OverflowPolicy.REROUTE, router_probs=p)
    assert over2 == over and int((m_ids == -1).sum()) == 0 and int(count_expert_assignments(m_ids, 8).max()) <= cap
    assert all(len(set(r)) == len(r) for r in m_ids.tolist())                        # no token got the same expert twice
    with pytest.raises(ExpertCapacityOverflow):
        apply_overflow_policy(ids, w, 8, cap, OverflowPolicy.ERROR)
    same = apply_overflow_policy(ids, w, 8, 1000, OverflowPolicy.ERROR)
    assert same[2] == 0 and same[0] is ids


def test_dynamic_capacity_follows_the_drop_rate():
    dc = DynamicCapacity(8, 2, DynamicCapacityConfig(initial_factor=1.0, window=4, target_drop_rate=0.01))
    for s in range(16):
        dc.update(_skewed(seed=s)[1])
    assert dc.current_factor > 1.3 and dc.get_stats()["adjustments"] >= 2
    uniform = torch.arange(64 * 2).view(64, 2) % 8
    hi = dc.current_factor
    for _ in range(12):
        dc.update(uniform)
    assert dc.current_factor < hi


def test_load_tracker_loss_and_entropy():
    E = 8
    uniform = torch.full((32, E), 1.0 / E)
    ids_u = (torch.arange(64).view(32, 2) % E)
    assert abs(float(load_balance_loss(uniform, ids_u, E)) - 1.0) < 1e-6
    assert abs(float(gate_entropy(uniform)) - 1.0) < 1e-6 and float(gate_entropy(torch.eye(E))) < 1e-6
    p, ids, w = _skewed()
    assert float(load_balance_loss(p, ids, E)) > 1.5
    tr = ExpertLoadTracker(LoadBalancingConfig(num_experts=E, top_k=2, ema_decay=0.5, dead_after_updates=3, z_loss_weight=1e-3))
    for s in range(6):
        pp, ii, _ = _skewed(seed=s)
        ii = torch.where(ii == 7, torch.zeros_like(ii), ii)             # expert 7 never gets a token
        tr.update(ii, pp)
    assert 0 in tr.get_hot_experts() and 7 in tr.get_cold_experts() and tr.get_dead_experts() == [7]
    assert tr.imbalance() > 2 and 0 < tr.entropy_ema < 1
    loss = tr.compute_loss(p, ids, router_logits=torch.log(p))
    assert float(loss) > 0


@pytest.mark.parametrize("strategy", list(PrefetchStrategy))
def test_prefetcher_predicts_and_loads_in_the_background(strategy):
    loaded = []

    def load(layer, expert):
        if expert == 5:
            raise RuntimeError("disk error")              # counted, never raised into the decode loop
        time.sleep(0.001)
        loaded.append((layer, expert))
        return {"layer": layer, "expert": expert}

    pf = ExpertPrefetcher(16, 2, load, PrefetchConfig(strategy=strategy, prefetch_k=3, history_window=8, min_confidence=0.0))
    pattern = [[1, 2], [3, 4], [1, 2], [3, 4], [1, 2], [3, 4], [1, 2]]      # period-2 routing: the next set is predictable
    preds = [pf.step(0, torch.tensor(ids), attention_pattern=[0.1, 0.8, 0.1]) for ids in pattern]
    pf.wait(5)
    assert preds[-1] and set(preds[-1]) <= {1, 2, 3, 4}
    if strategy in (PrefetchStrategy.MARKOV, PrefetchStrategy.ATTENTION_AWARE):
        assert set(preds[-1][:2]) == {3, 4}                                    # after {1, 2} always came {3, 4}
        assert pf.get_stats()["prediction_accuracy"] > 0.5
    assert all(pf.is_loaded(0, e) for e in preds[-1])
    st = pf.get_stats()
    assert st["requests"] >= st["hits"] + 1 and st["loaded"] == len(set(loaded)) and st["strategy"] == strategy.value
    assert pf.prefetch_experts(1, [5, 99, -1]) == 1                            # out-of-range ids are ignored, 5 is queued
    pf.wait(5)
    assert pf.get_stats()["failures"] == 1 and not pf.is_loaded(1, 5)
    assert pf.step(1, []) == []
    pf.stop()


def test_int8_router_matches_the_float_router():
    import torch
    from metal_marlin_b200 import ops
    from metal_marlin_b200.moe.router_int8 import (Int8Router, Int8RouterLinear, measure_quantization_error,
                                                   quantize_router_weights)
    torch.manual_seed(0)
    E, H, T = 64, 256, 200
    w = torch.randn(E, H) * 0.02
    x = torch.randn(T, H)
    q, s = quantize_router_weights(w)
    assert q.dtype == torch.int8 and s.shape == (E,) and int(q.abs().max()) == 127
    err = measure_quantization_error(w, x=x, topk=4)
    assert err["relative_error"] < 0.01 and err["topk_agreement"] > 0.9
    gate = Int8RouterLinear.from_weight(w)
    assert float((gate.dequantize(torch.float32) - q.float() * s.unsqueeze(1)).abs().max()) < 1e-3 * float(w.abs().max())
    lg = gate(x.bfloat16()).float()
    ref_lg = x.bfloat16().float() @ gate.dequantize(torch.float32).t()
    assert float((lg - ref_lg).abs().max()) < 0.02 * float(ref_lg.abs().max())
    # softmax top-4 with renormalisation and sigmoid + bias with group-limited choice: same experts as the float gate on
    # the de-quantized matrix except where two logits tie within bf16 rounding
    for kw in ({"topk": 4}, {"topk": 4, "scoring": 1, "n_group": 8, "topk_group": 4, "bias": torch.randn(E) * 0.01, "routed_scale": 1.8}):
        r = Int8Router(gate, **kw)
        ids, wts = r(x.bfloat16())
        ids2, wts2 = ops.moe_router(x.bfloat16().float(), gate.dequantize(torch.float32), **kw)
        same = (ids.sort(-1).values == ids2.sort(-1).values).all(-1)
        assert float(same.float().mean()) > 0.9 and ids.dtype == torch.int32
        a = torch.zeros(T, E).scatter_(1, ids.long(), wts)
        b = torch.zeros(T, E).scatter_(1, ids2.long(), wts2)
        assert float((a[same] - b[same]).abs().max()) < 0.02 * float(b.abs().max())
    counts = torch.zeros(E, dtype=torch.int32)
    Int8Router.from_weight(w, topk=2)(x.bfloat16(), counts=counts)
    assert int(counts.sum()) == 2 * T and r.num_experts == E and r.hidden_dim == H
