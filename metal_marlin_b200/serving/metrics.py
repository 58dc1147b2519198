"""Prometheus text metrics for the server, the MoE layers and the perplexity endpoint.

Parity: reference ``metal_marlin/serving/metrics.py:21-192`` (metric names), ``metal_marlin/trellis/metrics.py:194``
(``MoEMetrics``, gated by ``METAL_MARLIN_METRICS=1``) and ``metal_marlin/serving/perplexity.py:158``
(``PerplexityTracker``).  ``metal_marlin_throughput_tok_sec`` is added because the reference's own
acceptance script greps for it.
"""
from __future__ import annotations

import math
import statistics
import threading
import time
from collections import defaultdict, deque
from typing import Deque, Dict, List, Optional


def _quantile(xs: List[float], q: float) -> float:
    if not xs:
        return 0.0
    s = sorted(xs)
    i = min(len(s) - 1, max(0, int(math.ceil(q * len(s))) - 1))
    return s[i]


class MetricsCollector:
    def __init__(self, window: int = 2048):
        self._lock = threading.Lock()
        self.requests_total = 0
        self.active_requests = 0
        self.prompt_tokens = 0
        self.completion_tokens = 0
        self.by_endpoint: Dict[str, int] = defaultdict(int)
        self.errors_total: Dict[str, int] = defaultdict(int)
        self.latencies_ms: Deque[float] = deque(maxlen=window)
        self.ttft_ms: Deque[float] = deque(maxlen=window)
        self.queue_depth = 0
        self.gpu_memory_mb = 0.0
        self._tok_events: Deque = deque(maxlen=4096)
        self.started = time.time()

    def request_started(self, endpoint: str) -> float:
        with self._lock:
            self.requests_total += 1
            self.active_requests += 1
            self.by_endpoint[endpoint] += 1
        return time.perf_counter()

    def request_finished(self, t0: float, prompt_tokens: int = 0, completion_tokens: int = 0,
                         ttft_ms: Optional[float] = None, error: Optional[str] = None) -> None:
        with self._lock:
            self.active_requests = max(0, self.active_requests - 1)
            self.latencies_ms.append((time.perf_counter() - t0) * 1e3)
            self.prompt_tokens += prompt_tokens
            self.completion_tokens += completion_tokens
            if completion_tokens:
                self._tok_events.append((time.time(), completion_tokens))
            if ttft_ms is not None:
                self.ttft_ms.append(ttft_ms)
            if error:
                self.errors_total[error] += 1

    def throughput_tok_sec(self, horizon_s: float = 30.0) -> float:
        now = time.time()
        ev = [(t, n) for t, n in self._tok_events if now - t <= horizon_s]
        if not ev:
            return 0.0
        span = max(1e-3, now - min(t for t, _ in ev))
        return sum(n for _, n in ev) / span

    def latency_stats(self) -> dict:
        lat, tt = list(self.latencies_ms), list(self.ttft_ms)
        return {"total_ms": {q: _quantile(lat, v) for q, v in (("p50", .5), ("p95", .95), ("p99", .99))},
                "ttft_ms": {q: _quantile(tt, v) for q, v in (("p50", .5), ("p95", .95), ("p99", .99))},
                "count": len(lat)}

    def to_prometheus(self) -> str:
        with self._lock:
            lat = list(self.latencies_ms)
            n_req = max(1, self.requests_total)
            lines = [
                "# HELP metal_marlin_requests_total Total requests received", "# TYPE metal_marlin_requests_total counter",
                f"metal_marlin_requests_total {self.requests_total}",
                "# TYPE metal_marlin_active_requests gauge", f"metal_marlin_active_requests {self.active_requests}",
                "# TYPE metal_marlin_latency_ms summary",
            ]
            for q in (0.5, 0.95, 0.99):
                lines.append(f'metal_marlin_latency_ms{{quantile="{q}"}} {_quantile(lat, q):.3f}')
            for q in (0.5, 0.95, 0.99):
                lines.append(f'metal_marlin_ttft_ms{{quantile="{q}"}} {_quantile(list(self.ttft_ms), q):.3f}')
            lines += [
                "# TYPE metal_marlin_tokens_total counter",
                f'metal_marlin_tokens_total{{type="prompt"}} {self.prompt_tokens}',
                f'metal_marlin_tokens_total{{type="completion"}} {self.completion_tokens}',
                f"metal_marlin_avg_tokens_per_request {self.completion_tokens / n_req:.3f}",
            ]
            for ep, n in sorted(self.by_endpoint.items()):
                lines.append(f'metal_marlin_requests_by_endpoint{{endpoint="{ep}"}} {n}')
            for code, n in sorted(self.errors_total.items()):
                lines.append(f'metal_marlin_errors_total{{code="{code}"}} {n}')
            lines += [f"metal_marlin_gpu_memory_mb {self.gpu_memory_mb:.1f}", f"metal_marlin_queue_depth {self.queue_depth}",
                      f"metal_marlin_throughput_tok_sec {self.throughput_tok_sec():.3f}"]
        return "\n".join(lines) + "\n"


class MoEMetrics:
    """Counters of the MoE layers (forward time histogram, tokens, fast/fallback paths, NaNs)."""
    BUCKETS = (0.0005, 0.001, 0.0025, 0.005, 0.01, 0.025, 0.05, 0.1, 0.25, 1.0)

    def __init__(self):
        self.enabled = False
        self.reset()

    def reset(self):
        self.hist = [0] * (len(self.BUCKETS) + 1)
        self.sum_s = 0.0
        self.count = 0
        self.tokens = 0
        self.fast_path = 0
        self.fallback = 0
        self.nan_detected = 0
        self.memory_bytes = 0
        self.in_progress = 0
        self.expert_counts: Optional[List[int]] = None

    def observe(self, seconds: float, tokens: int, fast: bool = True) -> None:
        if not self.enabled:
            return
        for i, b in enumerate(self.BUCKETS):
            if seconds <= b:
                self.hist[i] += 1
                break
        else:
            self.hist[-1] += 1
        self.sum_s += seconds
        self.count += 1
        self.tokens += tokens
        if fast:
            self.fast_path += 1
        else:
            self.fallback += 1

    def to_prometheus(self) -> str:
        lines = ["# TYPE moe_forward_seconds histogram"]
        cum = 0
        for b, n in zip(self.BUCKETS, self.hist):
            cum += n
            lines.append(f'moe_forward_seconds_bucket{{le="{b}"}} {cum}')
        lines.append(f'moe_forward_seconds_bucket{{le="+Inf"}} {cum + self.hist[-1]}')
        lines += [f"moe_forward_seconds_sum {self.sum_s:.6f}", f"moe_forward_seconds_count {self.count}",
                  f"moe_tokens_processed_total {self.tokens}", f"moe_fast_path_used_total {self.fast_path}",
                  f"moe_fallback_total {self.fallback}", f"moe_nan_detected_total {self.nan_detected}",
                  f"moe_memory_bytes {self.memory_bytes}", f"moe_forward_in_progress {self.in_progress}"]
        return "\n".join(lines) + "\n"


moe_metrics = MoEMetrics()


class PerplexityTracker:
    def __init__(self, window: int = 100):
        self.values: Deque[float] = deque(maxlen=window)
        self.tokens_total = 0

    def record(self, ppl: float, tokens: int) -> None:
        self.values.append(ppl)
        self.tokens_total += tokens

    def stats(self) -> dict:
        v = list(self.values)
        if not v:
            return {"mean": 0.0, "median": 0.0, "min": 0.0, "max": 0.0, "samples": 0, "tokens_total": self.tokens_total}
        return {"mean": statistics.fmean(v), "median": statistics.median(v), "min": min(v), "max": max(v),
                "samples": len(v), "tokens_total": self.tokens_total}

    def to_prometheus(self) -> str:
        s = self.stats()
        return "".join(f"metal_marlin_perplexity_{k} {s[k]}\n" for k in ("mean", "median", "min", "max", "samples", "tokens_total"))
