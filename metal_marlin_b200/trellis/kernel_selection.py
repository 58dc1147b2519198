"""Run-time choice among the MoE execution paths for mixed-bit trellis experts, with feedback: a heuristic from the batch
size and the bit mix of the active experts, overridden by memory pressure, by skewed activation, by recorded timings, and
- with a benchmark callback - by occasional A/B runs whose outcomes are scored.

Paths (``ops.moe_forward`` / the generic MoE dispatch): ``slot_gemv`` - one streaming product per (token, slot), the decode path;
``grouped_gemv`` - rows sorted by expert, 8-row tiles on the streaming kernel; ``grouped_gemm`` - counting sort + tcgen05 grouped GEMM.
Families: experts of one bit width run as one bank launch (``uniform``), mostly-2-bit mixes favour the streaming paths longer
because their weights are half the bytes (``fast_2bit``), other mixes launch once per bit width (``mixed_bpw``).

Parity: reference ``trellis/kernel_selection_mixed.py`` (``MixedKernelSelector`` :275 with ``select_kernel`` / ``record_timing`` /
``get_statistics``, ``KernelFeedback`` :72, ``KernelABTester`` :102, ``get_kernel_for_batch_size`` :226) and ``trellis/optimizations.py``
(``ExpertSelectionCache`` :338, ``ExpertMemoryPool`` :431).
"""
from __future__ import annotations

import random
from collections import OrderedDict, deque
from dataclasses import dataclass, field
from typing import Callable, Deque, Dict, Iterable, List, Optional, Sequence, Set, Tuple

import torch

SLOT_GEMV, GROUPED_GEMV, GROUPED_GEMM = "slot_gemv", "grouped_gemv", "grouped_gemm"
ALL_KERNELS = (SLOT_GEMV, GROUPED_GEMV, GROUPED_GEMM)
UNIFORM_FAMILY, FAST_2BIT_FAMILY, MIXED_BPW_FAMILY = "uniform", "fast_2bit", "mixed_bpw"
STANDARD_FAMILY = UNIFORM_FAMILY


def get_kernel_for_batch_size(batch_size: int, slot_max: Optional[int] = None, grouped_max: Optional[int] = None) -> str:
    """The static rule of the op layer (its thresholds unless given)."""
    from .. import ops
    slot_max = ops.MOE_GEMV_MAX_T if slot_max is None else slot_max
    grouped_max = ops.MOE_GROUPED_GEMV_MAX_T if grouped_max is None else grouped_max
    return SLOT_GEMV if batch_size <= slot_max else GROUPED_GEMV if batch_size <= grouped_max else GROUPED_GEMM


def bit_family(active_expert_bits: Sequence[int]) -> str:
    bits = list(active_expert_bits)
    if not bits or len(set(bits)) == 1:
        return UNIFORM_FAMILY
    return FAST_2BIT_FAMILY if sum(1 for b in bits if b == 2) * 2 > len(bits) else MIXED_BPW_FAMILY


@dataclass
class KernelFeedback:
    kernel: str
    batch_size: int
    samples: Deque[float] = field(default_factory=deque)

    @property
    def mean_ms(self) -> float:
        return sum(self.samples) / len(self.samples) if self.samples else float("inf")


@dataclass
class ABResult:
    heuristic: str
    challenger: str
    heuristic_ms: float
    challenger_ms: float

    @property
    def winner(self) -> str:
        return self.challenger if self.challenger_ms < self.heuristic_ms else self.heuristic


class KernelABTester:
    """Times the heuristic's choice against one other candidate with a caller-supplied ``benchmark(kernel) -> ms``."""

    def __init__(self, rng: Optional[random.Random] = None):
        self.rng = rng or random
        self.results: List[ABResult] = []

    def run(self, heuristic: str, candidates: Iterable[str], benchmark: Callable[[str], float]) -> Optional[ABResult]:
        others = sorted(k for k in candidates if k != heuristic)
        if not others:
            return None
        challenger = self.rng.choice(others)
        res = ABResult(heuristic, challenger, float(benchmark(heuristic)), float(benchmark(challenger)))
        self.results.append(res)
        return res


class MixedKernelSelector:
    def __init__(self, history_len: int = 128, initial_exploration_rate: float = 0.05, min_feedback_samples: int = 3, rng: Optional[random.Random] = None):
        self.history_len, self.exploration_rate, self.min_feedback_samples = history_len, initial_exploration_rate, min_feedback_samples
        self.timings: Dict[Tuple[str, int], KernelFeedback] = {}
        self.ab = KernelABTester(rng)
        self.total_selections = self.correct_ab_selections = 0
        self.reasons: Dict[str, int] = {}

    # ------------------------------------------------------------------ rules
    @staticmethod
    def _bucket(batch_size: int) -> int:
        return 1 << max(0, int(batch_size) - 1).bit_length()               # timings are shared by batch sizes of one power-of-two bucket

    def _heuristic(self, batch_size: int, bits: Sequence[int]) -> Tuple[str, str]:
        fam = bit_family(bits)
        from .. import ops
        slot, grouped = ops.MOE_GEMV_MAX_T, ops.MOE_GROUPED_GEMV_MAX_T
        if fam == FAST_2BIT_FAMILY:                                        # half the bytes per weight: streaming stays ahead for twice the tokens
            slot, grouped = 2 * slot, 2 * grouped
        return get_kernel_for_batch_size(batch_size, slot, grouped), fam

    def _best_feedback(self, batch_size: int, available: Optional[Set[str]]) -> Optional[str]:
        b = self._bucket(batch_size)
        seen = {k: fb for (k, bb), fb in self.timings.items() if bb == b and len(fb.samples) >= self.min_feedback_samples
                and (available is None or k in available)}
        if len(seen) < 2:
            return None
        return min(seen, key=lambda k: seen[k].mean_ms)

    def select_kernel(self, batch_size: int, active_expert_bits: Sequence[int], use_fp32_acc: bool = False, available_kernels: Optional[Set[str]] = None,
                      gpu_memory_pressure: float = 0.0, expert_activation_pattern: Optional[Dict[str, float]] = None,
                      benchmark_kernel: Optional[Callable[[str], float]] = None) -> Tuple[str, Dict[str, object]]:
        """``(path, info)``; ``info["reason"]``: ``heuristic`` / ``memory_pressure`` (above 0.8 the grouped GEMM's gather / scatter workspaces are
        avoided) / ``activation_pattern_skewed`` (one expert takes 85 % of the tokens: the static rule is right) / ``feedback_optimization`` /
        ``availability_fallback`` / ``ab_testing_runtime``."""
        self.total_selections += 1
        baseline = get_kernel_for_batch_size(batch_size)
        choice, fam = self._heuristic(batch_size, active_expert_bits)
        info: Dict[str, object] = {"baseline_kernel": baseline, "heuristic_family": fam, "heuristic_kernel": choice, "reason": "heuristic"}

        def done(kernel: str, reason: str, **extra):
            self.reasons[reason] = self.reasons.get(reason, 0) + 1
            return kernel, {**info, "reason": reason, **extra}
        if use_fp32_acc and batch_size == 1:
            choice = baseline                                              # every path accumulates in fp32 here: nothing else to pick
        if gpu_memory_pressure > 0.8 and choice == GROUPED_GEMM:
            return done(GROUPED_GEMV, "memory_pressure")
        if expert_activation_pattern and expert_activation_pattern.get("top_expert_share", 0.0) >= 0.85:
            return done(baseline, "activation_pattern_skewed")
        fb = self._best_feedback(batch_size, available_kernels)
        if fb is not None and fb != choice:
            return done(fb, "feedback_optimization")
        if available_kernels is not None and choice not in available_kernels:
            return done(next((k for k in ALL_KERNELS if k in available_kernels), choice), "availability_fallback")
        if benchmark_kernel is not None and self.ab.rng.random() < self.exploration_rate:
            res = self.ab.run(choice, available_kernels or ALL_KERNELS, benchmark_kernel)
            if res is not None:
                self.record_timing(res.heuristic, batch_size, res.heuristic_ms, "ab")
                self.record_timing(res.challenger, batch_size, res.challenger_ms, "ab")
                self.correct_ab_selections += res.winner == choice
                return done(res.winner, "ab_testing_runtime", ab_test={"heuristic": res.heuristic, "challenger": res.challenger, "winner": res.winner,
                                                                       "heuristic_ms": res.heuristic_ms, "challenger_ms": res.challenger_ms})
        return done(choice, "heuristic")

    def record_timing(self, kernel: str, batch_size: int, ms: float, source: str = "runtime") -> None:
        key = (kernel, self._bucket(batch_size))
        fb = self.timings.get(key)
        if fb is None:
            fb = self.timings[key] = KernelFeedback(kernel, key[1], deque(maxlen=self.history_len))
        fb.samples.append(float(ms))

    @property
    def ab_tests_run(self) -> int:
        return len(self.ab.results)

    def get_statistics(self) -> Dict[str, object]:
        n = self.ab_tests_run
        return {"total_selections": self.total_selections, "ab_tests_run": n, "selection_accuracy": self.correct_ab_selections / n if n else 0.0,
                "exploration_rate": self.exploration_rate, "reasons": dict(self.reasons),
                "timings": {f"{k}@{b}": {"mean_ms": fb.mean_ms, "samples": len(fb.samples)} for (k, b), fb in self.timings.items()}}


def select_intelligent_kernel(batch_size: int, active_expert_bits: Sequence[int], selector: Optional[MixedKernelSelector] = None, **kw) -> str:
    return (selector or _DEFAULT).select_kernel(batch_size, active_expert_bits, **kw)[0]


_DEFAULT = MixedKernelSelector(initial_exploration_rate=0.0)


# ------------------------------------------------------------------------------------------------ routing cache, expert memory pool
class ExpertSelectionCache:
    """LRU of dispatch groupings keyed by the routing itself: decode steps often repeat the expert choice of the step before, and
    the grouping (sorted order, offsets) of an identical choice can be reused.  ``get(expert_ids)`` returns the cached grouping or
    None; ``put`` stores one.  Keys are the bytes of the id tensor, so a hit is exact."""

    def __init__(self, capacity: int = 64):
        self.capacity = capacity
        self._d: "OrderedDict[bytes, object]" = OrderedDict()
        self.hits = self.misses = 0

    @staticmethod
    def _key(expert_ids: torch.Tensor) -> bytes:
        t = expert_ids.detach().to("cpu", torch.int32).contiguous()
        return bytes(t.shape) + t.numpy().tobytes()

    def get(self, expert_ids: torch.Tensor):
        k = self._key(expert_ids)
        v = self._d.get(k)
        if v is None:
            self.misses += 1
            return None
        self.hits += 1
        self._d.move_to_end(k)
        return v

    def put(self, expert_ids: torch.Tensor, grouping) -> None:
        self._d[self._key(expert_ids)] = grouping
        self._d.move_to_end(self._key(expert_ids))
        while len(self._d) > self.capacity:
            self._d.popitem(last=False)

    def get_or_build(self, expert_ids: torch.Tensor, build: Callable[[torch.Tensor], object]):
        v = self.get(expert_ids)
        if v is None:
            v = build(expert_ids)
            self.put(expert_ids, v)
        return v

    def hit_rate(self) -> float:
        n = self.hits + self.misses
        return self.hits / n if n else 0.0

    def clear(self) -> None:
        self._d.clear()
        self.hits = self.misses = 0


class ExpertMemoryPool:
    """Reusable activation buffers for the MoE paths, bucketed by (rows rounded up to a power of two, width, dtype): a decode
    loop asks for the same few shapes every step, so after warm-up nothing is allocated."""

    def __init__(self, device=None, max_buffers_per_bucket: int = 4):
        self.device = torch.device(device) if device is not None else torch.device("cuda" if torch.cuda.is_available() else "cpu")
        self.max_per_bucket = max_buffers_per_bucket
        self._free: Dict[Tuple[int, int, torch.dtype], List[torch.Tensor]] = {}
        self.allocations = self.reuses = 0

    @staticmethod
    def _rows(n: int) -> int:
        return 1 << max(0, int(n) - 1).bit_length()

    def acquire(self, rows: int, width: int, dtype=torch.bfloat16) -> torch.Tensor:
        key = (self._rows(rows), int(width), dtype)
        pool = self._free.get(key)
        if pool:
            self.reuses += 1
            return pool.pop()[:rows]
        self.allocations += 1
        return torch.empty(key[0], width, dtype=dtype, device=self.device)[:rows]

    def release(self, t: torch.Tensor) -> None:
        base = t._base if t._base is not None else t
        key = (base.shape[0], base.shape[1], base.dtype)
        pool = self._free.setdefault(key, [])
        if len(pool) < self.max_per_bucket:
            pool.append(base)

    def stats(self) -> Dict[str, float]:
        held = sum(b.numel() * b.element_size() for p in self._free.values() for b in p)
        n = self.allocations + self.reuses
        return {"allocations": self.allocations, "reuses": self.reuses, "reuse_rate": self.reuses / n if n else 0.0, "bytes_held": held,
                "buckets": len(self._free)}

    def clear(self) -> None:
        self._free.clear()
