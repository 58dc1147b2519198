"""Reproducible decode benchmark: per-step latencies of a fixed workload, written as JSON with integrity hashes so that a
result can be tied to the exact model files, sources and built extension that produced it, and checked later.

    python bench/reproducible.py --preset glm-4.7-flash --num-steps 100 --output-json result.json
    python bench/reproducible.py --model-path path/to/model --num-steps 100 --output-json result.json
    python bench/reproducible.py --verify result.json

Specification: the prompt "The quick brown fox jumps over the lazy dog." (its token ids with a tokenizer, else a fixed id
sequence), batch 1, greedy; 3 warm-up decode steps, then N steps each bracketed by CUDA events on the launching stream (a
wall clock on CPU); mean, median, standard deviation, minimum, maximum and the 5th / 95th / 99th percentiles of the step
latency, with the matching tokens per second.  ``hashes``: sha-256 of the model files (or of the preset's configuration),
of the package sources and of the built extension; ``result_hash`` covers the specification, the hashes and the raw
per-step list, so editing any of them invalidates it.

Parity: reference ``bench_reproducible.py`` (same specification and statistics; integrity hashes over model and results).
"""
from __future__ import annotations

import argparse
import hashlib
import json
import math
import os
import platform
import statistics
import sys
import time
from typing import Dict, List, Optional

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

PROMPT = "The quick brown fox jumps over the lazy dog."
FALLBACK_IDS = [464, 2068, 7586, 21831, 18045, 625, 262, 16931, 3290, 13]
WARMUP_STEPS = 3


def sha256_file(path: str) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for chunk in iter(lambda: f.read(1 << 20), b""):
            h.update(chunk)
    return h.hexdigest()


def sha256_tree(root: str, suffixes=(".py", ".cu", ".cuh", ".cpp", ".h")) -> str:
    """One hash over the relative paths and contents of the source files below ``root`` (sorted, so it is stable)."""
    h = hashlib.sha256()
    for d, dirs, files in sorted(os.walk(root)):
        dirs[:] = sorted(x for x in dirs if x not in ("__pycache__", "_obj"))
        for f in sorted(files):
            if f.endswith(suffixes):
                p = os.path.join(d, f)
                h.update(os.path.relpath(p, root).encode())
                h.update(bytes.fromhex(sha256_file(p)))
    return h.hexdigest()


def canonical(obj) -> bytes:
    return json.dumps(obj, sort_keys=True, separators=(",", ":")).encode()


def percentile(xs: List[float], q: float) -> float:
    s = sorted(xs)
    if not s:
        return float("nan")
    k = (len(s) - 1) * q / 100.0
    lo, hi = math.floor(k), math.ceil(k)
    return s[lo] + (s[hi] - s[lo]) * (k - lo)


def summarize(ms: List[float]) -> Dict[str, Dict[str, float]]:
    lat = {"mean": statistics.fmean(ms), "median": statistics.median(ms), "std": statistics.pstdev(ms) if len(ms) > 1 else 0.0,
           "min": min(ms), "max": max(ms), "p5": percentile(ms, 5), "p95": percentile(ms, 95), "p99": percentile(ms, 99)}
    return {"latency_ms": {k: round(v, 4) for k, v in lat.items()},
            "tok_s": {k: round(1e3 / v, 2) for k, v in lat.items() if k != "std" and v > 0}}


def result_hash(doc: Dict) -> str:
    return hashlib.sha256(canonical({k: doc[k] for k in ("spec", "hashes", "step_ms")})).hexdigest()


def verify(path: str) -> bool:
    """True when the file's ``result_hash`` matches its specification, hashes and raw timings, and its statistics are the
    ones those timings give."""
    with open(path) as f:
        doc = json.load(f)
    return doc.get("result_hash") == result_hash(doc) and doc.get("stats") == summarize(doc["step_ms"])


def model_hash(model_path: Optional[str], preset: Optional[str]) -> Dict[str, str]:
    if model_path:
        files = sorted(f for f in os.listdir(model_path) if f.endswith((".safetensors", ".json")))
        h = hashlib.sha256()
        for f in files:
            h.update(f.encode())
            h.update(bytes.fromhex(sha256_file(os.path.join(model_path, f))))
        return {"model": h.hexdigest(), "model_files": str(len(files))}
    from metal_marlin_b200.models.config import get_preset
    return {"model": hashlib.sha256(canonical(get_preset(preset).to_dict())).hexdigest(), "model_files": "0 (random-init preset)"}


def run(model_path: Optional[str], preset: Optional[str], num_steps: int, device: Optional[str] = None, context: int = 4096,
        seed: int = 0) -> Dict:
    import torch
    from metal_marlin_b200.inference.decode import DecodeConfig, DecodeState, persistent_decode_step
    from metal_marlin_b200.inference.tokenizer import load_tokenizer
    from metal_marlin_b200.models.mmfp4_causal_lm import MMFP4ForCausalLM
    dev = device or ("cuda" if torch.cuda.is_available() else "cpu")
    lm = MMFP4ForCausalLM.from_pretrained(model_path, dev) if model_path else MMFP4ForCausalLM.from_config(preset, dev, seed)
    vocab = lm.config.vocab_size
    ids = None
    if model_path:
        try:
            ids = [int(t) for t in load_tokenizer(model_path, vocab).encode(PROMPT)]
        except Exception:
            ids = None
    if not ids:
        ids = [i % vocab for i in FALLBACK_IDS]
    state = DecodeState(lm, DecodeConfig(batch_size=1, max_context=context, max_new_tokens=num_steps + WARMUP_STEPS + 1))
    state.prefill([ids])
    cuda = dev.startswith("cuda")
    for _ in range(WARMUP_STEPS):
        persistent_decode_step(state)
    step_ms: List[float] = []
    if cuda:
        torch.cuda.synchronize()
        events = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(num_steps)]
        for a, b in events:
            a.record()
            persistent_decode_step(state)
            b.record()
        torch.cuda.synchronize()
        step_ms = [a.elapsed_time(b) for a, b in events]
    else:
        for _ in range(num_steps):
            t0 = time.perf_counter()
            persistent_decode_step(state)
            step_ms.append((time.perf_counter() - t0) * 1e3)
    pkg = os.path.join(ROOT, "metal_marlin_b200")
    so = os.path.join(pkg, "_C.so")
    doc = {
        "spec": {"prompt": PROMPT, "prompt_tokens": len(ids), "batch": 1, "sampling": "greedy", "warmup_steps": WARMUP_STEPS,
                 "num_steps": num_steps, "context": context, "model": model_path or f"preset:{preset}", "seed": seed,
                 "timer": "cuda events per step" if cuda else "perf_counter per step"},
        "hashes": {**model_hash(model_path, preset), "sources": sha256_tree(pkg),
                   "extension": sha256_file(so) if os.path.isfile(so) else "absent"},
        "environment": {"device": torch.cuda.get_device_name(0) if cuda else platform.processor() or "cpu", "torch": torch.__version__,
                        "cuda": torch.version.cuda, "python": platform.python_version(), "platform": platform.platform()},
        "step_ms": [round(x, 5) for x in step_ms],
    }
    doc["stats"] = summarize(doc["step_ms"])
    doc["result_hash"] = result_hash(doc)
    return doc


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--model-path")
    ap.add_argument("--preset", default=None)
    ap.add_argument("--num-steps", type=int, default=100)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--device", default=None)
    ap.add_argument("--output-json")
    ap.add_argument("--verify", metavar="JSON", help="check the integrity hash of a result file and exit")
    a = ap.parse_args(argv)
    if a.verify:
        ok = verify(a.verify)
        print(json.dumps({"file": a.verify, "valid": ok}))
        return 0 if ok else 1
    if not a.model_path and not a.preset:
        ap.error("give --model-path or --preset")
    doc = run(a.model_path, a.preset, a.num_steps, a.device, a.context)
    if a.output_json:
        with open(a.output_json, "w") as f:
            json.dump(doc, f, indent=1, sort_keys=True)
    print(json.dumps({"tok_s_median": doc["stats"]["tok_s"]["median"], "latency_ms": doc["stats"]["latency_ms"],
                      "result_hash": doc["result_hash"], "file": a.output_json}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
