"""Acceptance tracking and adaptive speculation depth.

Parity: reference ``metal_marlin/layers/adaptive_depth.py:26,90`` (``AdaptiveSpeculationController``: EMA of
the acceptance rate drives the draft length inside [1, 8], initial 4), ``metal_marlin/speculative/token_acceptance.py:107``
(``TokenAcceptanceTracker``) and ``metal_marlin/speculative/engine.py:667`` (``_update_num_spec``: raise above 0.8,
lower below 0.4 over a window of 10)."""
from __future__ import annotations

from collections import defaultdict, deque
from dataclasses import dataclass, field
from typing import Deque, Dict


@dataclass
class AdaptiveSpeculationController:
    min_depth: int = 1
    max_depth: int = 8
    depth: int = 4
    ema_alpha: float = 0.2
    increase_threshold: float = 0.8
    decrease_threshold: float = 0.4
    ema: float = 0.6
    steps: int = 0

    def update(self, proposed: int, accepted: int) -> int:
        if proposed > 0:
            rate = accepted / proposed
            self.ema = (1 - self.ema_alpha) * self.ema + self.ema_alpha * rate
            self.steps += 1
            if self.ema > self.increase_threshold and self.depth < self.max_depth:
                self.depth += 1
            elif self.ema < self.decrease_threshold and self.depth > self.min_depth:
                self.depth -= 1
        return self.depth


class TokenAcceptanceTracker:
    """Per-position and per-token acceptance statistics over a sliding window."""

    def __init__(self, window: int = 1000):
        self.events: Deque = deque(maxlen=window)
        self.by_position: Dict[int, list] = defaultdict(lambda: [0, 0])
        self.by_token: Dict[int, list] = defaultdict(lambda: [0, 0])
        self.total_proposed = self.total_accepted = 0

    def record(self, draft_tokens, num_accepted: int) -> None:
        for i, t in enumerate(draft_tokens):
            ok = i < num_accepted
            self.events.append(ok)
            self.by_position[i][0] += 1
            self.by_position[i][1] += ok
            self.by_token[int(t)][0] += 1
            self.by_token[int(t)][1] += ok
        self.total_proposed += len(draft_tokens)
        self.total_accepted += num_accepted

    @property
    def acceptance_rate(self) -> float:
        return self.total_accepted / max(1, self.total_proposed)

    @property
    def recent_rate(self) -> float:
        return sum(self.events) / max(1, len(self.events))

    def position_rates(self) -> Dict[int, float]:
        return {p: a / max(1, n) for p, (n, a) in sorted(self.by_position.items())}

    def expected_tokens_per_step(self) -> float:
        """1 (the verified/bonus token) + expected accepted drafts."""
        e, keep = 1.0, 1.0
        for p, r in self.position_rates().items():
            keep *= r
            e += keep
        return e
