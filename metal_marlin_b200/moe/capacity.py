"""Expert capacity: how many (token, slot) assignments one expert accepts per batch, what happens to the rest, and tools to
pick the capacity factor from observed routing.

``capacity = ceil(capacity_factor * tokens * top_k / num_experts)`` (at least ``min_capacity``).  Overflow policies:

* ``DROP``     the assignment is removed (id -1, weight 0); the token keeps its other experts' outputs
* ``RENORM``   as ``DROP``, and the surviving weights of the token are rescaled to their original sum
* ``REROUTE``  the assignment moves to the token's next-best expert that still has room (needs the router probabilities)
* ``ERROR``    raise ``ExpertCapacityOverflow`` (what an expert-parallel exchange with fixed receive buffers reports)

Parity: reference ``metal_marlin/capacity.py``: ``OverflowInfo`` ``:48``, ``CapacityStats`` ``:90``, ``CapacityAnalyzer`` ``:145``,
``compute_expert_capacity`` ``:261``, ``count_expert_assignments`` ``:287``, ``analyze_overflow_rate`` ``:306``,
``auto_tune_capacity`` ``:342``, ``DynamicCapacityConfig`` ``:414``, ``DynamicCapacity`` ``:440``.
"""
from __future__ import annotations

import enum
import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch


class OverflowPolicy(enum.Enum):
    DROP = "drop"
    RENORM = "renorm"
    REROUTE = "reroute"
    ERROR = "error"


def compute_expert_capacity(num_tokens: int, num_experts: int, top_k: int, capacity_factor: float = 1.25, min_capacity: int = 1) -> int:
    return max(min_capacity, int(math.ceil(capacity_factor * num_tokens * top_k / max(1, num_experts))))


def count_expert_assignments(expert_ids: torch.Tensor, num_experts: int) -> torch.Tensor:
    flat = expert_ids.reshape(-1).long()
    return torch.bincount(flat[flat >= 0], minlength=num_experts)


@dataclass
class OverflowInfo:
    """One batch: assignments, capacity, and what did not fit."""
    num_tokens: int
    capacity: int
    counts: torch.Tensor                      # [E] assignments per expert
    dropped: int
    overflow_experts: List[int] = field(default_factory=list)

    @property
    def total(self) -> int:
        return int(self.counts.sum())

    @property
    def drop_rate(self) -> float:
        return self.dropped / self.total if self.total else 0.0

    @property
    def utilization(self) -> float:
        """Fraction of the reserved capacity (``E x capacity`` rows) that holds a real assignment."""
        E = self.counts.numel()
        return float(self.counts.clamp(max=self.capacity).sum()) / max(1, E * self.capacity)


@dataclass
class CapacityStats:
    batches: int = 0
    total_assignments: int = 0
    total_dropped: int = 0
    overflow_batches: int = 0
    per_expert_overflow: Dict[int, int] = field(default_factory=dict)
    peak_load: int = 0

    @property
    def overall_drop_rate(self) -> float:
        return self.total_dropped / self.total_assignments if self.total_assignments else 0.0

    @property
    def overflow_rate(self) -> float:
        return self.overflow_batches / self.batches if self.batches else 0.0

    def top_overflow_experts(self, k: int = 10) -> List[Tuple[int, int]]:
        return sorted(self.per_expert_overflow.items(), key=lambda kv: -kv[1])[:k]


class CapacityAnalyzer:
    """Feed it the routing of every batch; it reports how often and where a given capacity factor would overflow."""

    def __init__(self, num_experts: int, top_k: int, capacity_factor: float = 1.25, min_capacity: int = 1, history: int = 256):
        self.num_experts, self.top_k, self.capacity_factor, self.min_capacity = num_experts, top_k, capacity_factor, min_capacity
        self.history = history
        self.reset()

    def compute_capacity(self, num_tokens: int) -> int:
        return compute_expert_capacity(num_tokens, self.num_experts, self.top_k, self.capacity_factor, self.min_capacity)

    def record_batch(self, expert_ids: torch.Tensor) -> OverflowInfo:
        T = expert_ids.shape[0]
        cap = self.compute_capacity(T)
        counts = count_expert_assignments(expert_ids, self.num_experts)
        over = (counts - cap).clamp_min(0)
        info = OverflowInfo(T, cap, counts, int(over.sum()), over.nonzero().reshape(-1).tolist())
        s = self.stats
        s.batches += 1
        s.total_assignments += info.total
        s.total_dropped += info.dropped
        s.overflow_batches += int(info.dropped > 0)
        s.peak_load = max(s.peak_load, int(counts.max()) if counts.numel() else 0)
        for e in info.overflow_experts:
            s.per_expert_overflow[e] = s.per_expert_overflow.get(e, 0) + int(over[e])
        self._hist.append(info)
        if len(self._hist) > self.history:
            self._hist.pop(0)
        return info

    def get_stats(self) -> CapacityStats:
        return self.stats

    def get_batch_history(self) -> List[OverflowInfo]:
        return list(self._hist)

    def reset(self) -> None:
        self.stats = CapacityStats()
        self._hist: List[OverflowInfo] = []


def analyze_overflow_rate(batches: Sequence[torch.Tensor], num_experts: int, top_k: int, factors: Sequence[float] = (1.0, 1.25, 1.5, 2.0)
                          ) -> Dict[float, Dict[str, float]]:
    """Drop rate and share of overflowing batches for each candidate capacity factor over recorded routing decisions."""
    out = {}
    for f in factors:
        an = CapacityAnalyzer(num_experts, top_k, f)
        for ids in batches:
            an.record_batch(ids)
        out[f] = {"drop_rate": an.stats.overall_drop_rate, "overflow_rate": an.stats.overflow_rate, "peak_load": an.stats.peak_load}
    return out


def auto_tune_capacity(batches: Sequence[torch.Tensor], num_experts: int, top_k: int, target_drop_rate: float = 0.01,
                       lo: float = 1.0, hi: float = 8.0, tol: float = 0.01) -> float:
    """Smallest capacity factor (to ``tol``) whose drop rate over the recorded batches stays at or below the target."""
    def rate(f):
        return analyze_overflow_rate(batches, num_experts, top_k, (f,))[f]["drop_rate"]
    if rate(hi) > target_drop_rate:
        return hi
    while hi - lo > tol:
        mid = 0.5 * (lo + hi)
        if rate(mid) <= target_drop_rate:
            hi = mid
        else:
            lo = mid
    return hi


@dataclass
class DynamicCapacityConfig:
    initial_factor: float = 1.25
    min_factor: float = 1.0
    max_factor: float = 4.0
    target_drop_rate: float = 0.01
    window: int = 32                 # batches per adjustment
    step_up: float = 1.15
    step_down: float = 0.95


class DynamicCapacity:
    """Capacity factor that follows the observed drop rate: raised quickly when drops exceed the target, lowered slowly when a
    whole window shows none (reserved rows cost memory and sweep time in a grouped GEMM)."""

    def __init__(self, num_experts: int, top_k: int, config: Optional[DynamicCapacityConfig] = None):
        self.num_experts, self.top_k, self.cfg = num_experts, top_k, config or DynamicCapacityConfig()
        self.reset()

    @property
    def current_factor(self) -> float:
        return self._factor

    def get_capacity(self, num_tokens: int) -> int:
        return compute_expert_capacity(num_tokens, self.num_experts, self.top_k, self._factor)

    def update(self, expert_ids: torch.Tensor) -> float:
        cap = self.get_capacity(expert_ids.shape[0])
        counts = count_expert_assignments(expert_ids, self.num_experts)
        self._dropped += int((counts - cap).clamp_min(0).sum())
        self._total += int(counts.sum())
        self._n += 1
        if self._n >= self.cfg.window:
            self._maybe_adjust()
        return self._factor

    def _maybe_adjust(self) -> None:
        c = self.cfg
        rate = self._dropped / self._total if self._total else 0.0
        if rate > c.target_drop_rate:
            self._factor = min(c.max_factor, self._factor * c.step_up)
            self.adjustments += 1
        elif rate == 0.0 and self._factor > c.min_factor:
            self._factor = max(c.min_factor, self._factor * c.step_down)
            self.adjustments += 1
        self.last_drop_rate = rate
        self._dropped = self._total = self._n = 0

    def reset(self) -> None:
        self._factor = self.cfg.initial_factor
        self._dropped = self._total = self._n = 0
        self.adjustments = 0
        self.last_drop_rate = 0.0

    def get_stats(self) -> dict:
        return {"factor": self._factor, "adjustments": self.adjustments, "last_drop_rate": self.last_drop_rate}


def apply_overflow_policy(expert_ids: torch.Tensor, weights: torch.Tensor, num_experts: int, capacity: int,
                          policy: OverflowPolicy = OverflowPolicy.DROP, router_probs: Optional[torch.Tensor] = None
                          ) -> Tuple[torch.Tensor, torch.Tensor, int]:
    """Enforce ``capacity`` assignments per expert (earliest tokens win).  Returns ``(ids, weights, overflowed)`` where
    ``overflowed`` counts the assignments that did not fit their first-choice expert."""
    policy = OverflowPolicy(policy)
    T, k = expert_ids.shape
    flat = expert_ids.reshape(-1).long()
    onehot = torch.nn.functional.one_hot(flat.clamp_min(0), num_experts) * (flat >= 0).unsqueeze(1)
    rank = (onehot.cumsum(0) * onehot).sum(1)                       # 1-based arrival order within the expert
    keep = ((rank <= capacity) & (flat >= 0)).view(T, k)
    over = int(((flat >= 0).view(T, k) & ~keep).sum())
    if over == 0:
        return expert_ids, weights, 0
    if policy is OverflowPolicy.ERROR:
        from ..parallel.health import ExpertCapacityOverflow
        raise ExpertCapacityOverflow(f"{over} assignments exceed the expert capacity of {capacity}")
    ids = torch.where(keep, expert_ids, torch.full_like(expert_ids, -1))
    w = torch.where(keep, weights, torch.zeros_like(weights))
    if policy is OverflowPolicy.RENORM:
        tot, left = weights.sum(-1, keepdim=True), w.sum(-1, keepdim=True)
        w = torch.where(left > 0, w * tot / left.clamp_min(1e-30), w)
    elif policy is OverflowPolicy.REROUTE:
        if router_probs is None:
            raise ValueError("REROUTE needs the router probabilities")
        load = count_expert_assignments(ids, num_experts)
        order = router_probs.argsort(-1, descending=True)
        for t, s in (~keep & (expert_ids >= 0)).nonzero().tolist():      # overflow is rare: a host loop over the few cases
            taken = set(int(e) for e in ids[t].tolist() if e >= 0)
            for e in order[t].tolist():
                if e not in taken and load[e] < capacity:
                    ids[t, s] = e
                    w[t, s] = weights[t, s]
                    load[e] += 1
                    break
    return ids, w, over
