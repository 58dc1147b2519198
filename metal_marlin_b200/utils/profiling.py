"""Call-level profiling switches and statistics under the reference's names (``enable_profiling`` / ``disable_profiling`` /
``is_profiling_enabled``, ``get_profile_records`` / ``get_profile_stats`` / ``get_all_profile_stats`` / ``clear_profiles`` /
``print_profile_summary``, ``ProfileRecord`` / ``ProfileStats``) over the kernel timer of ``profiling/roofline.py`` (its
``@profile_kernel`` decorator times a call with the device synchronised when profiling is on).  Parity: reference
``metal_marlin/utils/profiling.py:47-218``."""
from __future__ import annotations

import statistics
from dataclasses import dataclass
from typing import Dict, List

from ..profiling import roofline as _rf
from ..profiling.roofline import profile_kernel          # noqa: F401  (re-export)


@dataclass
class ProfileRecord:
    wall_time_ms: float
    name: str = ""


@dataclass
class ProfileStats:
    name: str
    count: int
    total_ms: float
    mean_ms: float
    min_ms: float
    max_ms: float
    std_ms: float


def enable_profiling() -> None:
    _rf.PROFILE_ON = True


def disable_profiling() -> None:
    _rf.PROFILE_ON = False


def is_profiling_enabled() -> bool:
    return bool(_rf.PROFILE_ON)


def get_profile_records(name: str) -> List[ProfileRecord]:
    return [ProfileRecord(s * 1e3, name) for s in _rf.profile_records().get(name, [])]


def get_profile_stats(name: str) -> ProfileStats:
    ms = [s * 1e3 for s in _rf.profile_records().get(name, [])]
    if not ms:
        return ProfileStats(name, 0, 0.0, 0.0, 0.0, 0.0, 0.0)
    return ProfileStats(name, len(ms), sum(ms), statistics.fmean(ms), min(ms), max(ms), statistics.pstdev(ms) if len(ms) > 1 else 0.0)


def get_all_profile_stats() -> Dict[str, ProfileStats]:
    return {k: get_profile_stats(k) for k in _rf.profile_records()}


def clear_profiles() -> None:
    _rf.profile_records().clear()


def print_profile_summary(out=print) -> None:
    rows = sorted(get_all_profile_stats().values(), key=lambda s: -s.total_ms)
    out(f"{'kernel':40s} {'calls':>6s} {'total ms':>10s} {'mean ms':>9s} {'max ms':>9s}")
    for s in rows:
        out(f"{s.name[:40]:40s} {s.count:6d} {s.total_ms:10.3f} {s.mean_ms:9.4f} {s.max_ms:9.4f}")
