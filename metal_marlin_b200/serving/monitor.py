"""Terminal monitor for a running server: polls ``/metrics`` (Prometheus text) and ``/health`` and prints request, token,
latency, queue and memory figures with rates between polls.

    python -m metal_marlin_b200 monitor --url http://127.0.0.1:8000 [--interval 2] [--once]

Parity: reference ``scripts/inference_monitor.py`` (terminal dashboard over the server's metrics endpoint).
"""
from __future__ import annotations

import json
import re
import time
import urllib.request
from typing import Dict, Optional, Tuple

_LINE = re.compile(r"^([a-zA-Z_:][a-zA-Z0-9_:]*)(\{[^}]*\})?\s+([-+0-9.eEinfNa]+)\s*$")


def parse_metrics(text: str) -> Dict[str, float]:
    """``name`` or ``name{labels}`` -> value for every sample line of a Prometheus exposition."""
    out: Dict[str, float] = {}
    for line in text.splitlines():
        if not line or line.startswith("#"):
            continue
        m = _LINE.match(line.strip())
        if not m:
            continue
        try:
            out[m.group(1) + (m.group(2) or "")] = float(m.group(3))
        except ValueError:
            pass
    return out


def _get(metrics: Dict[str, float], name: str, label: Optional[str] = None, default: float = 0.0) -> float:
    if label is None:
        return metrics.get(name, default)
    for k, v in metrics.items():
        if k.startswith(name + "{") and label in k:
            return v
    return default


def render(metrics: Dict[str, float], prev: Optional[Dict[str, float]] = None, dt: float = 0.0, health: Optional[dict] = None) -> str:
    """A fixed-width table; with a previous sample and the time between them, request and token rates are added."""
    def rate(name, label=None):
        if prev is None or dt <= 0:
            return None
        return (_get(metrics, name, label) - _get(prev, name, label)) / dt
    rows = [("status", (health or {}).get("status", "?")),
            ("requests total / active", f"{_get(metrics, 'metal_marlin_requests_total'):.0f} / {_get(metrics, 'metal_marlin_active_requests'):.0f}"),
            ("queue depth", f"{_get(metrics, 'metal_marlin_queue_depth'):.0f}"),
            ("tokens prompt / completion", f"{_get(metrics, 'metal_marlin_tokens_total', 'prompt'):.0f} / "
                                           f"{_get(metrics, 'metal_marlin_tokens_total', 'completion'):.0f}"),
            ("latency ms p50 / p95 / p99", " / ".join(f"{_get(metrics, 'metal_marlin_latency_ms', q):.1f}" for q in ('"0.5"', '"0.95"', '"0.99"'))),
            ("throughput tok/s (server)", f"{_get(metrics, 'metal_marlin_throughput_tok_sec'):.1f}"),
            ("gpu memory MB", f"{_get(metrics, 'metal_marlin_gpu_memory_mb'):.0f}")]
    r = rate("metal_marlin_requests_total")
    if r is not None:
        rows.append(("requests/s since last poll", f"{r:.2f}"))
        rows.append(("completion tok/s since last poll", f"{rate('metal_marlin_tokens_total', 'completion'):.1f}"))
    if "metal_marlin_perplexity_mean" in metrics:
        rows.append(("perplexity mean", f"{metrics['metal_marlin_perplexity_mean']:.3f}"))
    if "moe_tokens_processed_total" in metrics:
        rows.append(("MoE tokens / fallbacks", f"{metrics['moe_tokens_processed_total']:.0f} / {metrics.get('moe_fallback_total', 0):.0f}"))
    w = max(len(k) for k, _ in rows)
    return "\n".join(f"{k.ljust(w)}  {v}" for k, v in rows)


def fetch(url: str, timeout: float = 5.0) -> Tuple[Dict[str, float], dict]:
    with urllib.request.urlopen(url.rstrip("/") + "/metrics", timeout=timeout) as r:
        metrics = parse_metrics(r.read().decode("utf-8", "replace"))
    try:
        with urllib.request.urlopen(url.rstrip("/") + "/health", timeout=timeout) as r:
            health = json.loads(r.read().decode("utf-8", "replace"))
    except Exception:
        health = {}
    return metrics, health


def run(url: str, interval: float = 2.0, once: bool = False, out=print, polls: Optional[int] = None, fetch_fn=fetch) -> int:
    prev, t_prev, n = None, 0.0, 0
    while True:
        try:
            metrics, health = fetch_fn(url)
        except Exception as e:
            out(f"[{time.strftime('%H:%M:%S')}] {url}: {e}")
            if once:
                return 1
            metrics = None
        now = time.monotonic()
        if metrics is not None:
            out(f"--- {url}  {time.strftime('%H:%M:%S')} ---\n" + render(metrics, prev, now - t_prev, health))
            prev, t_prev = metrics, now
        n += 1
        if once or (polls is not None and n >= polls):
            return 0
        time.sleep(interval)
