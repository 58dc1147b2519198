"""LRU cache of device-resident experts for MoE models whose experts live in host memory (offload), with hit-rate
statistics and frequency-aware prefetch hints.  Parity: reference ``metal_marlin/expert_cache.py`` and the 16-entry
de-quantization cache of ``metal_marlin/glm4_moe_experts.py:140-215``."""
from __future__ import annotations

from collections import Counter, OrderedDict
from typing import Callable, Dict, Hashable, List, Optional, Tuple


class ExpertCache:
    def __init__(self, capacity: int, loader: Callable[[Hashable], object], on_evict: Optional[Callable[[Hashable, object], None]] = None):
        """``loader(key)`` brings an expert to the device; ``key`` is typically ``(layer, expert)``."""
        self.capacity, self.loader, self.on_evict = capacity, loader, on_evict
        self._d: "OrderedDict[Hashable, object]" = OrderedDict()
        self.hits = self.misses = self.evictions = 0
        self.freq: Counter = Counter()

    def get(self, key: Hashable):
        self.freq[key] += 1
        if key in self._d:
            self.hits += 1
            self._d.move_to_end(key)
            return self._d[key]
        self.misses += 1
        val = self.loader(key)
        self._d[key] = val
        while len(self._d) > self.capacity:
            k, v = self._d.popitem(last=False)
            self.evictions += 1
            if self.on_evict:
                self.on_evict(k, v)
        return val

    def prefetch(self, keys) -> int:
        n = 0
        for k in keys:
            if k not in self._d:
                self.get(k)
                self.hits, self.misses = self.hits, self.misses - 1     # prefetches are not demand misses
                n += 1
        return n

    def hot_keys(self, n: int) -> List[Hashable]:
        return [k for k, _ in self.freq.most_common(n)]

    def hit_rate(self) -> float:
        t = self.hits + self.misses
        return self.hits / t if t else 0.0

    def __contains__(self, key) -> bool:
        return key in self._d

    def __len__(self) -> int:
        return len(self._d)
