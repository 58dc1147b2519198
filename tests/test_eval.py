"""Evaluation utilities (reference: tests/test_perplexity.py, test_accuracy.py, test_moe_routing_analysis.py)."""
import math

import torch

from metal_marlin_b200.eval import (ExpertUsageProfiler, apply_capacity, kl_divergence, load_balancing_loss, quality_report,
                                    sliding_window_nll, synthetic_corpus)


def _uniform_fn(V):
    return lambda ids: torch.zeros(len(ids), V)


def test_sliding_window_perplexity_of_uniform_model_is_vocab_size():
    ids = synthetic_corpus(50, 300, seed=1)
    r = sliding_window_nll(_uniform_fn(50), ids, max_length=64, stride=32)
    assert abs(r["perplexity"] - 50.0) < 1e-3 and r["tokens"] == 299


def test_windows_score_every_token_once():
    V = 11
    calls = []

    def fn(ids):
        calls.append(len(ids))
        lg = torch.full((len(ids), V), -10.0)
        for i in range(len(ids) - 1):
            lg[i, ids[i + 1]] = 10.0              # a perfect model
        return lg

    r = sliding_window_nll(fn, list(range(10)) * 13, max_length=40, stride=16)
    assert r["tokens"] == 129 and r["nll"] < 1e-6 and max(calls) <= 40


def test_kl_and_quality_report():
    torch.manual_seed(0)
    W = torch.randn(20, 20)
    ref = lambda ids: W[torch.tensor(ids)]
    noisy = lambda ids: W[torch.tensor(ids)] + 0.05 * torch.randn(len(ids), 20, generator=torch.Generator().manual_seed(1))
    ids = synthetic_corpus(20, 200)
    same = kl_divergence(ref, ref, ids)
    assert same["kl_mean"] < 1e-9 and same["top1_agreement"] == 1.0
    q = quality_report(ref, noisy, ids, max_length=64, stride=32)
    assert 0 < q["kl_mean"] < 0.05 and q["top1_agreement"] > 0.8 and abs(q["perplexity_delta_pct"]) < 20


def test_expert_usage_and_capacity():
    prof = ExpertUsageProfiler(1, 4)
    ids = torch.tensor([[0, 1], [0, 2], [0, 1], [0, 3]])
    probs = torch.full((4, 4), 0.25)
    prof.record(0, ids, probs)
    s = prof.summary()
    assert s["hottest"] == [0] and s["dead_experts"] == [0] and abs(s["gate_entropy"][0] - math.log(4)) < 1e-9
    assert abs(s["load_imbalance"][0] - 2.0) < 1e-9 and int(prof.coact[0, 0, 1]) == 2
    new_ids, w, dropped = apply_capacity(ids, torch.ones(4, 2), 4, capacity_factor=1.0)
    assert dropped == 2 and new_ids[:, 0].tolist() == [0, 0, -1, -1] and float(w[2, 0]) == 0.0
    assert float(load_balancing_loss(probs, ids, 4)) == 1.0
