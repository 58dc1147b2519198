"""NaN guard: run a fast path, check its output, fall back to a slow reference path when it produced non-finite
values, and keep statistics.  Parity: reference ``metal_marlin/trellis/nan_guard.py:152`` (stats ``:35``)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch


@dataclass
class NaNStats:
    calls: int = 0
    nan_detected: int = 0
    fallbacks: int = 0
    unrecovered: int = 0


class NaNGuard:
    def __init__(self, check_every: int = 1, sanitize: bool = True):
        self.check_every, self.sanitize = max(1, check_every), sanitize
        self.stats = NaNStats()

    def run(self, fast: Callable[[], torch.Tensor], slow: Optional[Callable[[], torch.Tensor]] = None) -> torch.Tensor:
        self.stats.calls += 1
        y = fast()
        if self.stats.calls % self.check_every:
            return y
        if bool(torch.isfinite(y).all()):
            return y
        self.stats.nan_detected += 1
        if slow is not None:
            self.stats.fallbacks += 1
            y = slow()
            if bool(torch.isfinite(y).all()):
                return y
        self.stats.unrecovered += 1
        return torch.nan_to_num(y, nan=0.0, posinf=0.0, neginf=0.0) if self.sanitize else y
