"""Kernel-selection auto-tuner on a modelled timer (no GPU): crossover search, table export / import, installation into
``ops`` and the online adapter.  Parity: reference ``tests/test_autotune_mixed_bpw.py`` (tuner with mocked benchmarks,
JSON round trip, lookup)."""
import dataclasses

import pytest
import torch

from metal_marlin_b200 import autotune as at
from metal_marlin_b200 import ops


def test_crossover_is_monotone():
    b = (1, 2, 4, 8, 16)
    assert at.crossover(b, [1, 1, 1, 1, 9], [2, 2, 2, 2, 2]) == 8
    assert at.crossover(b, [3, 1, 1, 1, 1], [2, 2, 2, 2, 2]) == 0          # a later win does not count after a loss
    assert at.crossover(b, [1, 1, 1, 1, 1], [2, 2, 2, 2, 2]) == 16
    assert at.crossover(b, [2.05, 9, 9, 9, 9], [2, 2, 2, 2, 2], tolerance=0.03) == 1


class _ModelTimer:
    """Times a closure by what ``ops`` would dispatch to: streaming kernels cost per token, tensor-core kernels a fixed
    launch plus a small per-token term."""

    def __init__(self, tokens_of):
        self.tokens_of = tokens_of

    def __call__(self, fn):
        t = self.tokens_of()
        if ops.GEMV_MAX_M >= at._BIG or ops.MOE_GEMV_MAX_T >= at._BIG:
            return 4.0 + 1.0 * t                   # per-row streaming
        if ops.MOE_GROUPED_GEMV_MAX_T >= at._BIG:
            return 12.0 + 0.5 * t                  # expert-sorted streaming
        return 40.0 + 0.05 * t                     # tensor cores


def test_tune_linear_and_install(tmp_path):
    state = {"t": 0}
    tuner = at.KernelAutoTuner(device="cpu", timer=_ModelTimer(lambda: state["t"]), batch_sizes=(1, 8, 16, 32, 48, 64))

    real = torch.randn

    def randn(m, *a, **k):          # the tuner draws an activation per token count: record it for the timer
        state["t"] = m
        return real(m, *a, **k)
    torch.randn = randn
    try:
        limits = tuner.tune_linear([(256, 128), (128, 256)], group_size=64)
    finally:
        torch.randn = real
    # 4 + t <= (40 + 0.05 t) * 1.03  ->  t <= 39
    assert limits == {"256x128": 32, "128x256": 32}
    assert tuner.config.thresholds["GEMV_MAX_M"] == 32
    assert ops.GEMV_MAX_M == 32 and ops.GEMV_LIMITS == {}              # overrides were undone
    path = str(tmp_path / "t" / "tuning.json")
    tuner.export_config(path)
    cfg = at.TunedConfig.load(path)
    assert cfg.linear_limits == limits and len(cfg.measurements) == 12
    cfg.linear_limits["256x128"] = 48
    old = (ops.GEMV_MAX_M, dict(ops.GEMV_LIMITS), list(ops.MOE_TOKEN_TILES))
    try:
        assert at.apply_config(cfg) == {"GEMV_MAX_M": 32}
        assert at.get_optimal_config(40, 256, 128) == {"kernel": "fp4_gemv", "limit": 48, "tuned": True}
        assert at.get_optimal_config(40, 128, 256)["kernel"] == "fp4_gemm_tcgen05"
        assert at.get_optimal_config(40, 512, 512) == {"kernel": "fp4_gemm_tcgen05", "limit": 32, "tuned": False}
        W = at._random_fp4(256, 128, 64, "cpu")
        assert ops._gemv_limit(W) == 48
    finally:
        ops.GEMV_MAX_M, ops.GEMV_LIMITS, ops.MOE_TOKEN_TILES = old


def test_tune_moe_thresholds():
    state = {"t": 0}
    tuner = at.KernelAutoTuner(device="cpu", timer=_ModelTimer(lambda: state["t"]), batch_sizes=(1, 8, 16, 32, 64, 128))
    real = torch.randn

    def randn(m, *a, **k):
        state["t"] = m
        return real(m, *a, **k)
    torch.randn = randn
    try:
        slot_max, sorted_max = tuner.tune_moe(hidden=128, inter=64, num_experts=8, topk=2, group_size=64, token_tiles=(32, 64))
    finally:
        torch.randn = real
    # per-slot streaming (4 + t) beats sorted streaming (12 + t / 2) up to 16 tokens; sorted beats the GEMM (40 + t / 20) up to 64
    assert (slot_max, sorted_max) == (16, 64)
    assert tuner.config.thresholds == {"MOE_GEMV_MAX_T": 16, "MOE_GROUPED_GEMV_MAX_T": 64}
    assert set(tuner.config.moe_token_tiles) == {"16", "32", "64", "128"}
    assert (ops.MOE_GEMV_MAX_T, ops.MOE_GROUPED_GEMV_MAX_T) == (8, 128)               # overrides were undone


def test_load_config_from_environment(tmp_path, monkeypatch):
    cfg = at.TunedConfig(device="x", thresholds={"FMHA_MIN_T": 384, "NOT_A_THRESHOLD": 1}, moe_token_tiles={"64": 32, "512": 128})
    path = str(tmp_path / "tuning.json")
    cfg.save(path)
    monkeypatch.setenv("MMB200_TUNING_FILE", path)
    old = (ops.FMHA_MIN_T, dict(ops.GEMV_LIMITS), list(ops.MOE_TOKEN_TILES))
    try:
        got = at.load_config()
        assert got.thresholds["FMHA_MIN_T"] == 384 and ops.FMHA_MIN_T == 384
        assert not hasattr(ops, "NOT_A_THRESHOLD")
        assert ops.MOE_TOKEN_TILES == [(64, 32), (512, 128)]
    finally:
        ops.FMHA_MIN_T, ops.GEMV_LIMITS, ops.MOE_TOKEN_TILES = old
    monkeypatch.setenv("MMB200_TUNING_FILE", str(tmp_path / "absent.json"))
    assert at.load_config() is None


def test_online_adapter_switches_to_the_faster_variant():
    ad = at.OnlineAdapter(("graph", "eager"), min_samples=2, reprobe_every=10)
    seen = []
    for step in range(40):
        v = ad.choose("bs8")
        seen.append(v)
        us = {"graph": 100.0, "eager": 150.0}[v] if step < 20 else {"graph": 300.0, "eager": 150.0}[v]
        ad.observe("bs8", v, us)
    assert seen[:4].count("graph") == 2 and seen[:4].count("eager") == 2      # both sampled first
    assert ad.best("bs8") == "eager"                                          # graph became slower, the average followed
    assert seen[5] == "graph" and seen[-2] == "eager" and seen[-1] == "graph"       # the 40th call re-probes the slower one
    assert ad.best("unknown") is None
