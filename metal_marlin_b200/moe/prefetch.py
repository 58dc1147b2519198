"""Predictive expert prefetching for models whose expert banks do not all fit on the device (``memory/expert_cache.py`` holds
the resident set, ``memory/streaming.py`` moves the bytes): after every MoE layer's routing decision the prefetcher predicts
which experts the next token will route to and loads them in a background pool, so the demand miss - a host-to-device copy on
the critical path - becomes a hit.

Strategies: ``TOP_K_RECENCY`` (experts seen most recently in this layer, decayed by age), ``FREQUENCY`` (most frequent over
the history window), ``MARKOV`` (first-order transitions: which experts followed the current set last time),
``ATTENTION_AWARE`` (Markov scores reweighted by how much attention mass the current token puts on recent positions: a token
attending to its neighbourhood tends to reuse their experts).

Parity: reference ``metal_marlin/moe/prefetch.py``: ``PrefetchStrategy`` ``:16``, ``PrefetchConfig`` ``:26``, ``ExpertPrefetcher``
``:41`` (``start`` / ``stop`` / ``step`` / ``prefetch_experts`` / ``get_stats``; failures are counted, never raised).
"""
from __future__ import annotations

import enum
import threading
from collections import Counter, defaultdict, deque
from concurrent.futures import Future, ThreadPoolExecutor
from dataclasses import dataclass
from typing import Any, Callable, Deque, Dict, Iterable, List, Optional, Sequence, Tuple


class PrefetchStrategy(str, enum.Enum):
    TOP_K_RECENCY = "top_k_recency"
    FREQUENCY = "frequency"
    MARKOV = "markov"
    ATTENTION_AWARE = "attention_aware"


@dataclass
class PrefetchConfig:
    strategy: PrefetchStrategy = PrefetchStrategy.TOP_K_RECENCY
    prefetch_k: int = 4
    history_window: int = 32
    decay_factor: float = 0.9
    min_confidence: float = 0.05
    async_threads: int = 2
    enable_stats: bool = True
    max_prefetch_queue: int = 16
    max_loaded: int = 256               # loaded entries kept reachable (oldest dropped first)


class ExpertPrefetcher:
    """``load_fn(layer, expert)`` brings one expert to the device (typically ``ExpertCache.get`` on ``(layer, expert)``)."""

    def __init__(self, num_experts: int, num_layers: int, load_fn: Callable[[int, int], Any], config: Optional[PrefetchConfig] = None,
                 cache: Any = None):
        self.num_experts, self.num_layers, self.load_fn, self.cache = num_experts, num_layers, load_fn, cache
        self.config = config or PrefetchConfig()
        w = max(1, self.config.history_window)
        self._history: Dict[int, Deque[Tuple[int, ...]]] = defaultdict(lambda: deque(maxlen=w))
        self._trans: Dict[int, Dict[int, Counter]] = defaultdict(lambda: defaultdict(Counter))      # layer -> expert -> next experts
        self._futures: List[Future] = []
        self._loaded: "dict[Tuple[int, int], Any]" = {}
        self._lock = threading.Lock()
        self._executor: Optional[ThreadPoolExecutor] = None
        self.requests = self.hits = self.misses = self.failures = self.predicted = self.predicted_right = 0
        self._last_pred: Dict[int, List[int]] = {}

    # ------------------------------------------------------------------ lifecycle
    def start(self) -> None:
        if self._executor is None:
            self._executor = ThreadPoolExecutor(max_workers=max(1, self.config.async_threads), thread_name_prefix="expert-prefetch")

    def stop(self) -> None:
        ex, self._executor = self._executor, None
        if ex is not None:
            ex.shutdown(wait=False, cancel_futures=True)

    def wait(self, timeout: Optional[float] = None) -> None:
        """Block until the queued loads have finished (tests, orderly shutdown)."""
        for f in list(self._futures):
            try:
                f.result(timeout)
            except Exception:
                pass

    # ------------------------------------------------------------------ prediction
    @staticmethod
    def _ids(x) -> List[int]:
        if hasattr(x, "reshape"):
            x = x.reshape(-1).tolist()
        return sorted({int(e) for e in x if int(e) >= 0})

    def _scores(self, layer: int, current: Sequence[int], attention: Optional[Sequence[float]] = None) -> Dict[int, float]:
        c, hist = self.config, self._history[layer]
        s: Dict[int, float] = defaultdict(float)
        strat = PrefetchStrategy(c.strategy)
        if strat is PrefetchStrategy.TOP_K_RECENCY:
            for age, ids in enumerate(reversed(hist)):
                for e in ids:
                    s[e] += c.decay_factor ** age
        elif strat is PrefetchStrategy.FREQUENCY:
            for ids in hist:
                for e in ids:
                    s[e] += 1.0
        else:
            tr = self._trans[layer]
            for e in current:
                tot = sum(tr[e].values())
                for nxt, n in tr[e].items():
                    s[nxt] += n / tot
            if strat is PrefetchStrategy.ATTENTION_AWARE and attention is not None and len(hist):
                # attention[i]: mass on the i-th most recent position; its experts are likely to be reused
                for age, ids in enumerate(reversed(hist)):
                    if age < len(attention):
                        for e in ids:
                            s[e] += float(attention[age])
            if not s:                                   # nothing learned yet: fall back to recency
                for age, ids in enumerate(reversed(hist)):
                    for e in ids:
                        s[e] += c.decay_factor ** age
        tot = sum(s.values())
        return {e: v / tot for e, v in s.items()} if tot > 0 else {}

    def predict(self, layer: int, current: Iterable[int], attention: Optional[Sequence[float]] = None) -> List[int]:
        sc = self._scores(layer, list(current), attention)
        ranked = sorted(sc.items(), key=lambda kv: (-kv[1], kv[0]))
        return [e for e, v in ranked if v >= self.config.min_confidence][: self.config.prefetch_k]

    # ------------------------------------------------------------------ per-step hook
    def step(self, layer: int, current_indices, attention_pattern: Optional[Sequence[float]] = None) -> List[int]:
        """Record this token's routing for ``layer`` and queue loads for the predicted next-token experts."""
        ids = self._ids(current_indices)
        if not ids:
            return []
        with self._lock:
            last = self._last_pred.get(layer)
            if last is not None and self.config.enable_stats:
                self.predicted += len(last)
                self.predicted_right += len(set(last) & set(ids))
            hist = self._history[layer]
            if hist:
                for prev in hist[-1]:
                    for e in ids:
                        self._trans[layer][prev][e] += 1
            hist.append(tuple(ids))
            pred = self.predict(layer, ids, attention_pattern)
            self._last_pred[layer] = pred
        self.prefetch_experts(layer, pred)
        return pred

    def prefetch_experts(self, layer: int, expert_ids: Sequence[int]) -> int:
        if not expert_ids:
            return 0
        self.start()
        queued = 0
        with self._lock:
            self._futures = [f for f in self._futures if not f.done()]
            pending = {getattr(f, "_key", None) for f in self._futures}
            room = max(0, self.config.max_prefetch_queue - len(self._futures))
            for e in list(expert_ids)[:room]:
                if not 0 <= e < self.num_experts:
                    continue
                key = (layer, int(e))
                self.requests += 1
                if key in self._loaded:
                    self.hits += 1
                    continue
                self.misses += 1
                if key in pending:
                    continue
                fut = self._executor.submit(self._load, key)
                fut._key = key
                self._futures.append(fut)
                queued += 1
        return queued

    def _load(self, key: Tuple[int, int]):
        try:
            val = self.load_fn(*key)
        except Exception:
            with self._lock:
                self.failures += 1
            return None
        with self._lock:
            self._loaded[key] = val
            while len(self._loaded) > self.config.max_loaded:
                self._loaded.pop(next(iter(self._loaded)))
        return val

    def is_loaded(self, layer: int, expert: int) -> bool:
        return (layer, expert) in self._loaded

    def get_stats(self) -> dict:
        return {"requests": self.requests, "hits": self.hits, "misses": self.misses, "failures": self.failures,
                "hit_rate": self.hits / self.requests if self.requests else 0.0,
                "prediction_accuracy": self.predicted_right / self.predicted if self.predicted else 0.0,
                "loaded": len(self._loaded), "strategy": PrefetchStrategy(self.config.strategy).value}
