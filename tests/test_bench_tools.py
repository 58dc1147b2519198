"""Benchmark drivers run end to end on CPU with tiny models (reference: tests/validation/test_e2e_validation.py)."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(args, timeout=600):
    r = subprocess.run([sys.executable] + args, cwd=ROOT, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=timeout)
    assert r.returncode == 0, r.stdout[-3000:]
    return json.loads([l for l in r.stdout.splitlines() if l.startswith("{")][-1])


def test_serving_load_generator_completes_all_requests():
    out = _run(["bench/serving_load.py", "--model", "tiny-mla-moe", "--rate", "100", "--requests", "10", "--prompt-min", "8", "--prompt-max", "40",
                "--out-min", "4", "--out-max", "10", "--kv-blocks", "256", "--device", "cpu"])
    assert out["completed"] == 10 and out["ttft_ms_p50"] > 0 and out["latency_ms_p99"] >= out["latency_ms_p50"] and out["output_tok_s"] > 0


def test_config_runner_and_reference_arm():
    out = _run(["bench/run_configs.py", "--config", "1"])
    assert out["config"] == 1 and out["tokens"] == 32
    r = subprocess.run([sys.executable, "bench/run_configs.py", "--list"], cwd=ROOT, stdout=subprocess.PIPE, text=True)
    assert r.returncode == 0 and "[5]" in r.stdout
    ref = _run(["bench.py", "--impl", "reference"])
    assert ref["impl"] == "reference" and "unavailable" in ref


import pytest


@pytest.mark.gpu
def test_tp_gemm_chain_emulated_on_one_gpu():
    """GEMM with scatter epilogue -> reduce with fused residual add + RMSNorm -> GEMM with the gather wait in its TMA
    producer, ranks emulated as buffers of one GPU: numerics of every stage against fp32 PyTorch, status word clean."""
    out = _run(["-m", "metal_marlin_b200.profiling.tp_gemm_bench", "--tokens", "300", "--out", "512", "--inner", "1024", "--tp", "2",
                "--iters", "2"])
    assert out["status"] == 0
    assert out["rel_err"] < 2e-2 and out["rel_err_norm"] < 2e-2 and out["rel_err_ag_gemm"] < 2e-2
