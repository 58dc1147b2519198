"""Reproducible benchmark (``bench/reproducible.py``) on a tiny preset on CPU: document layout, statistics, and the
integrity hash that detects edited timings.  Parity: reference ``bench_reproducible.py`` (JSON with integrity hashes)."""
import importlib.util
import json
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
spec = importlib.util.spec_from_file_location("bench_reproducible", os.path.join(ROOT, "bench", "reproducible.py"))
rep = importlib.util.module_from_spec(spec)
spec.loader.exec_module(rep)


def test_statistics_and_percentiles():
    s = rep.summarize([1.0, 2.0, 3.0, 4.0])
    assert s["latency_ms"]["mean"] == 2.5 and s["latency_ms"]["median"] == 2.5 and s["latency_ms"]["min"] == 1.0
    assert s["latency_ms"]["p5"] == 1.15 and s["latency_ms"]["p95"] == 3.85
    assert s["tok_s"]["median"] == 400.0 and "std" not in s["tok_s"]


def test_run_writes_a_verifiable_document(tmp_path):
    out = str(tmp_path / "r.json")
    assert rep.main(["--preset", "tiny-llama", "--num-steps", "5", "--context", "64", "--device", "cpu", "--output-json", out]) == 0
    doc = json.load(open(out))
    assert len(doc["step_ms"]) == 5 and doc["spec"]["warmup_steps"] == 3 and doc["spec"]["batch"] == 1
    assert set(doc["hashes"]) == {"model", "model_files", "sources", "extension"} and len(doc["hashes"]["sources"]) == 64
    assert doc["stats"]["tok_s"]["median"] > 0 and rep.verify(out)
    # the same sources and preset hash the same way; an edited timing breaks the result hash
    assert doc["hashes"]["sources"] == rep.sha256_tree(os.path.join(ROOT, "metal_marlin_b200"))
    doc["step_ms"][0] /= 2
    json.dump(doc, open(out, "w"))
    assert not rep.verify(out)
    assert rep.main(["--verify", out]) == 1
