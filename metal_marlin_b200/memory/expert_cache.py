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


class TileCoordinator:
    """Tile arithmetic over one expert matrix ``[out_features, in_features]``: linear tile index <-> (row tile, column
    tile) <-> element ranges, in the device layout of the FP4 weights by default (16 output rows x 64 input columns per
    tile, ``qtile[out / 16, in / 64, 32, 4]``), so partial-expert prefetch and cache code can name the bytes of a tile.
    Parity: reference ``metal_marlin/expert_cache.py:628`` (``TileCoordinator``)."""

    def __init__(self, weight_shape: Tuple[int, int], tile_shape: Tuple[int, int] = (16, 64)):
        self.weight_shape, self.tile_shape = tuple(weight_shape), tuple(tile_shape)
        self.num_row_tiles = -(-weight_shape[0] // tile_shape[0])
        self.num_col_tiles = -(-weight_shape[1] // tile_shape[1])
        self.num_tiles = self.num_row_tiles * self.num_col_tiles

    def tile_to_coords(self, tile_idx: int) -> Tuple[int, int]:
        if not 0 <= tile_idx < self.num_tiles:
            raise IndexError(tile_idx)
        return divmod(tile_idx, self.num_col_tiles)

    def coords_to_tile(self, row_tile: int, col_tile: int) -> int:
        if not (0 <= row_tile < self.num_row_tiles and 0 <= col_tile < self.num_col_tiles):
            raise IndexError((row_tile, col_tile))
        return row_tile * self.num_col_tiles + col_tile

    def tile_bounds(self, tile_idx: int) -> Tuple[slice, slice]:
        """Element ranges ``(rows, cols)`` of a tile, clipped at the matrix edge."""
        r, c = self.tile_to_coords(tile_idx)
        th, tw = self.tile_shape
        return (slice(r * th, min((r + 1) * th, self.weight_shape[0])), slice(c * tw, min((c + 1) * tw, self.weight_shape[1])))

    def tiles_for_rows(self, row0: int, row1: int) -> List[int]:
        """Tiles that hold any of the output rows ``[row0, row1)`` (a row-sharded or partially fetched expert)."""
        th = self.tile_shape[0]
        return [self.coords_to_tile(r, c) for r in range(row0 // th, -(-row1 // th)) for c in range(self.num_col_tiles)]

    def tile_nbytes(self, bits: int = 4) -> int:
        return self.tile_shape[0] * self.tile_shape[1] * bits // 8

    def byte_offset(self, tile_idx: int, bits: int = 4) -> int:
        """Offset of a tile inside a matrix stored tile after tile (row tiles outermost)."""
        return tile_idx * self.tile_nbytes(bits)

    def iter_tiles(self):
        for i in range(self.num_tiles):
            yield (i, *self.tile_to_coords(i))


class ExpertWeightStreamer:
    """Device residency of routed experts under a budget: ``get_expert_weights(e)`` returns the resident copy, loading it on a
    miss (``loader(e)`` brings the expert's tensors to the device; without a loader a record ``{"expert_idx", "resident"}`` stands
    in, which is enough for the bookkeeping and for tests); eviction takes, among the least recently used half, the expert
    with the fewest accesses, and halves its count so that a formerly hot expert can cool down; ``predicted_experts`` ranks
    the non-resident experts of the recent routing history for prefetching.  Reference ``expert_weight_streaming.py:22``."""

    def __init__(self, num_experts: int = 256, gpu_cache_size: int = 64, loader: Optional[Callable[[int], object]] = None,
                 on_evict: Optional[Callable[[int, object], None]] = None, history: int = 1024):
        import collections
        self.num_experts, self.gpu_cache_size = num_experts, gpu_cache_size
        self.loader, self.on_evict = loader, on_evict
        self.gpu_cache: "OrderedDict[int, object]" = OrderedDict()
        self.access_counts: Dict[int, int] = collections.defaultdict(int)
        self._history = collections.deque(maxlen=history)
        self.hits = self.misses = self.evictions = 0

    def _load(self, e: int) -> None:
        self.gpu_cache[e] = self.loader(e) if self.loader is not None else {"expert_idx": e, "resident": True}
        self.evict_cold()

    def prefetch_experts(self, expert_indices) -> int:
        n = 0
        for e in expert_indices:
            if 0 <= e < self.num_experts and e not in self.gpu_cache:
                self._load(int(e))
                n += 1
        return n

    def get_expert_weights(self, expert_idx: int):
        if not 0 <= expert_idx < self.num_experts:
            raise ValueError(f"expert_idx {expert_idx} out of range [0, {self.num_experts})")
        self.access_counts[expert_idx] += 1
        self._history.append(expert_idx)
        if expert_idx in self.gpu_cache:
            self.hits += 1
            self.gpu_cache.move_to_end(expert_idx)
            return self.gpu_cache[expert_idx]
        self.misses += 1
        self._load(expert_idx)
        return self.gpu_cache[expert_idx]

    def evict_cold(self) -> None:
        while len(self.gpu_cache) > self.gpu_cache_size:
            order = list(self.gpu_cache)
            newest = order[-1]
            pool = [e for e in order[: max(1, len(order) // 2)] if e != newest] or order[:1]
            victim = min(pool, key=lambda e: self.access_counts[e])
            obj = self.gpu_cache.pop(victim)
            self.access_counts[victim] //= 2
            self.evictions += 1
            if self.on_evict is not None:
                self.on_evict(victim, obj)

    def predicted_experts(self, top_k: int = 8, window: int = 256) -> List[int]:
        freq: Dict[int, int] = {}
        for e in list(self._history)[-window:]:
            if e not in self.gpu_cache:
                freq[e] = freq.get(e, 0) + 1
        return sorted(freq, key=lambda e: (-freq[e], e))[:top_k]

    def hit_rate(self) -> float:
        n = self.hits + self.misses
        return self.hits / n if n else 0.0
