"""MoE routing profiler: statistics against a direct count, co-occurrence, next-layer predictability, reports, log files,
and the capture-hook driver on a tiny MoE model."""
import json
import math
import os

import numpy as np
import pytest
import torch

from metal_marlin_b200.analysis import (ExpertCooccurrence, ExpertLoadStats, LayerRoutingProfile, MoERoutingProfiler, RoutingPredictability,
                                        analyze_routing_from_file, profile_model, simulate_routing_for_model)
from metal_marlin_b200.analysis.moe_routing import gini, main


def test_layer_statistics_match_direct_counts():
    rs = np.random.RandomState(0)
    E, K, T = 6, 2, 200
    ids = np.stack([rs.choice(5, size=K, replace=False, p=[0.5, 0.2, 0.15, 0.1, 0.05]) for _ in range(T)])      # expert 5 never fires
    probs = rs.rand(T, K).astype(np.float32)
    p = MoERoutingProfiler(E, 2, K)
    p.record_routing(0, ids[:120], probs[:120])
    p.record_routing(0, torch.from_numpy(ids[120:]).reshape(-1), torch.from_numpy(probs[120:]))       # flat ids are cut into rows of top_k
    prof = p.layer_profiles[0]
    counts = np.bincount(ids.reshape(-1), minlength=E)
    assert prof.total_tokens == T and prof.active_experts == 5 and prof.dead_experts == 1 and prof.get_dead_experts() == [5]
    for e in range(E):
        s = prof.expert_stats[e]
        assert s.total_activations == counts[e] and s.activation_rate == pytest.approx(counts[e] / (T * K))
        assert s.rank_distribution == {k: int((ids[:, k] == e).sum()) for k in range(K)}
        if counts[e]:
            sel = probs[ids == e]
            assert s.avg_probability == pytest.approx(float(sel.mean()), abs=1e-6) and s.std_probability == pytest.approx(float(sel.std()), abs=1e-5)
            assert s.primary_selection_rate == pytest.approx((ids[:, 0] == e).sum() / counts[e])
    rate = counts / counts.sum()
    assert prof.entropy == pytest.approx(-sum(r * math.log2(r) for r in rate if r > 0)) and prof.load_balance_cv == pytest.approx(counts.std() / counts.mean())
    assert prof.gini_coefficient == pytest.approx(gini(counts)) and gini(np.ones(4)) == pytest.approx(0.0) and gini(np.array([0, 0, 0, 8.])) == pytest.approx(0.75)
    assert 0 in prof.get_hot_experts() and set(prof.get_cold_experts()) <= {3, 4} and prof.get_hot_experts(threshold=100.0) == []
    assert p.layer_profiles[1].total_tokens == 0 and p.get_dead_experts() == [5] and p.get_dead_experts(0) == [5]
    co = p.cooccurrence
    direct = np.zeros((E, E), dtype=np.int64)
    for a, b in ids:
        direct[a, b] += 1
        direct[b, a] += 1
    assert np.array_equal(co.cooccurrence_matrix, direct) and co.top_pairs[0][2] == direct.max()
    i, j, _ = co.top_pairs[0]
    assert co.conditional_probs[i, j] == pytest.approx(direct[i, j] / counts[i])
    assert p.get_prefetch_recommendations(0, 2) == list(np.argsort(-counts, kind="stable")[:2])
    with pytest.raises(ValueError):
        p.record_routing(2, ids)
    with pytest.raises(ValueError):
        p.record_routing(0, np.array([[0, 9]]))
    p.record_routing(1, np.array([[0, -1], [1, 2]]))          # negative ids (padding) are ignored
    assert p.layer_profiles[1].expert_stats[0].total_activations == 1 and sum(s.total_activations for s in p.layer_profiles[1].expert_stats.values()) == 3


def test_predictability_from_transitions():
    E, K, T = 8, 1, 400
    g = torch.Generator().manual_seed(0)
    a = torch.randint(0, E, (T, K), generator=g)
    det = MoERoutingProfiler(E, 3, K, predictability_threshold=0.9)
    det.record_routing(0, a)
    det.record_routing(1, (a + 3) % E)                               # fully decided by the layer before
    det.record_routing(2, torch.randint(0, E, (T, K), generator=g))  # independent
    pr = det.predictability
    assert pr.per_layer_accuracy[1] == pytest.approx(1.0) and pr.per_layer_accuracy[2] < 0.35 and pr.predictable_from_layer == -1
    assert det.get_prefetch_recommendations(1, 1, given_previous=[2]) == [5]
    assert pr.layer_correlations.shape == (3, 3) and pr.layer_correlations[0, 0] == pytest.approx(1.0)
    ok = MoERoutingProfiler(E, 2, K, predictability_threshold=0.9)
    ok.record_routing(0, a)
    ok.record_routing(1, (a + 1) % E)
    assert ok.predictability.predictable_from_layer == 0 and ok.predictability.avg_prediction_accuracy == pytest.approx(1.0)
    # a new pass does not pair the last layer of one pass with the first of the next; differing token counts are not paired either
    ok.end_pass()
    ok.record_routing(1, a[:10])
    assert set(ok._trans) == {1} and int(ok._trans[1].sum()) == T


def test_reports_heatmap_log_and_cli(tmp_path, capsys):
    p = simulate_routing_for_model("mixtral", num_samples=300, seed=1)
    rep = p.generate_report()
    assert rep["config"]["num_experts"] == 8 and rep["summary"]["layers_profiled"] == 32 and len(rep["layers"]) == 32
    assert rep["layers"]["0"]["dead_experts"] >= 1 and 0 < rep["predictability"]["avg_prediction_accuracy"] <= 1
    uncoupled = simulate_routing_for_model("mixtral", num_samples=300, seed=1, layer_coupling=0.0)
    assert p.predictability.avg_prediction_accuracy > uncoupled.predictability.avg_prediction_accuracy
    out = tmp_path / "r" / "report.json"
    p.save_report(str(out))
    assert json.loads(out.read_text())["summary"] == rep["summary"]
    img = p.plot_routing_heatmap(str(tmp_path / "h.png"), cell=4)
    assert img.shape == (32 * 4, 8 * 4, 3) and img.dtype == np.uint8 and os.path.getsize(tmp_path / "h.png") > 0
    p.plot_routing_heatmap(str(tmp_path / "h.ppm"))
    assert (tmp_path / "h.ppm").read_bytes().startswith(b"P6 48 192 255\n")
    assert "32 layers x 8 experts" in p.summary_text()
    with pytest.raises(ValueError):
        simulate_routing_for_model("no-such-model")
    log = tmp_path / "routing.jsonl"
    with open(log, "w") as f:
        f.write(json.dumps({"layer": 0, "expert_ids": [[0, 1], [2, 1]], "probs": [[0.7, 0.3], [0.6, 0.4]]}) + "\n\n")
        f.write(json.dumps({"layer": 1, "expert_ids": [[3, 1], [3, 0]]}) + "\n")
    q = analyze_routing_from_file(str(log), 4, 2, 2, output_dir=str(tmp_path / "o"))
    assert q.layer_profiles[0].expert_stats[1].total_activations == 2 and q.layer_profiles[0].expert_stats[0].avg_probability == pytest.approx(0.7)
    assert q.layer_profiles[1].expert_stats[3].avg_probability == 0.0 and os.path.isfile(tmp_path / "o" / "routing_report.json")
    assert os.path.isfile(tmp_path / "o" / "routing_heatmap.png")
    assert main(["--log", str(log), "--num-experts", "4", "--num-layers", "2"]) == 0 and main(["--simulate", "glm47", "--samples", "50"]) == 0
    assert "MoE routing" in capsys.readouterr().out
    for cls in (ExpertCooccurrence, ExpertLoadStats, LayerRoutingProfile, RoutingPredictability):
        assert cls is not None
    assert ExpertCooccurrence(3).cooccurrence_matrix.shape == (3, 3) and RoutingPredictability(2).layer_correlations.shape == (2, 2)


def test_profile_model_through_capture_hook():
    from metal_marlin_b200.models.mmfp4_causal_lm import MMFP4ForCausalLM
    lm = MMFP4ForCausalLM.from_config("tiny-qwen3-moe", "cpu", 0)
    cfg = lm.config
    g = torch.Generator().manual_seed(0)
    seqs = [torch.randint(0, cfg.vocab_size, (12,), generator=g).tolist() for _ in range(2)]
    p = profile_model(lm, seqs)
    profs = [pr for pr in p.layer_profiles.values() if pr.total_tokens]
    assert len(profs) >= 1 and all(pr.total_tokens == 24 for pr in profs)
    assert all(sum(s.total_activations for s in pr.expert_stats.values()) == 24 * cfg.num_experts_per_tok for pr in profs)
    if len(profs) > 1:
        assert 1 in p.predictability.per_layer_accuracy
