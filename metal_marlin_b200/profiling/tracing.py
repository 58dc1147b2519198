"""Chrome-trace event recording and launch tracing, env-gated so they cost nothing when off.

Parity: reference ``metal_marlin/tracing.py`` (``MM_TRACE=1``; ``record_event`` ``:29``, ``trace_scope`` ``:70``,
``trace_kernel`` ``:90``, ``write_trace`` ``:110``) and ``metal_marlin/launch_tracing.py`` (``MM_LAUNCH_TRACE=1``;
``record_dispatch / commit / wait / copy / kernel`` ``:64-140``, ``trace_region`` ``:146``, counters ``:181-211``,
``write_json`` ``:222``).  Kernel launches are counted at the op registry (``ops.launch_count``); with tracing on,
``trace_scope`` also opens an NVTX range so the same regions show up in vendor profilers.
"""
from __future__ import annotations

import contextlib
import json
import os
import threading
import time
from collections import Counter
from typing import Dict, List, Optional

import torch

TRACE_ON = os.environ.get("MM_TRACE", "0") == "1"
LAUNCH_TRACE_ON = os.environ.get("MM_LAUNCH_TRACE", "0") == "1"
_events: List[dict] = []
_lock = threading.Lock()
_t0 = time.perf_counter()


def enable(trace: bool = True, launches: bool = True) -> None:
    global TRACE_ON, LAUNCH_TRACE_ON
    TRACE_ON, LAUNCH_TRACE_ON = trace, launches


def _now_us() -> float:
    return (time.perf_counter() - _t0) * 1e6


def record_event(name: str, ts_us: float, dur_us: float, cat: str = "host", args: Optional[dict] = None, tid: Optional[int] = None) -> None:
    if not TRACE_ON:
        return
    with _lock:
        _events.append({"name": name, "cat": cat, "ph": "X", "ts": ts_us, "dur": dur_us, "pid": os.getpid(),
                        "tid": tid if tid is not None else threading.get_ident() % 100000, "args": args or {}})


@contextlib.contextmanager
def trace_scope(name: str, cat: str = "host", sync: bool = False, **args):
    """Time a host region (optionally synchronising the device on both sides so the span covers the GPU work)."""
    if not TRACE_ON:
        yield
        return
    if sync and torch.cuda.is_available():
        torch.cuda.synchronize()
    nvtx = torch.cuda.is_available()
    if nvtx:
        torch.cuda.nvtx.range_push(name)
    t = _now_us()
    try:
        yield
    finally:
        if sync and torch.cuda.is_available():
            torch.cuda.synchronize()
        if nvtx:
            torch.cuda.nvtx.range_pop()
        record_event(name, t, _now_us() - t, cat, args)


@contextlib.contextmanager
def trace_kernel(name: str, **args):
    """Device-timed span: CUDA events on the current stream (resolved when the trace is written)."""
    if not TRACE_ON or not torch.cuda.is_available():
        yield
        return
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t = _now_us()
    e0.record()
    try:
        yield
    finally:
        e1.record()
        with _lock:
            _events.append({"name": name, "cat": "kernel", "ph": "X", "ts": t, "_ev": (e0, e1), "pid": os.getpid(), "tid": 1, "args": args})


def write_trace(path: str) -> int:
    """Write the Chrome trace (``chrome://tracing`` / Perfetto).  Returns the number of events."""
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    out = []
    with _lock:
        for e in _events:
            e = dict(e)
            ev = e.pop("_ev", None)
            if ev is not None:
                e["dur"] = ev[0].elapsed_time(ev[1]) * 1e3
            out.append(e)
    with open(path, "w") as f:
        json.dump({"traceEvents": out, "displayTimeUnit": "ms"}, f)
    return len(out)


def clear() -> None:
    with _lock:
        _events.clear()


# ------------------------------------------------------------------------------------------ launch tracing
class LaunchTracer:
    """Counts kernel launches, host<->device copies, synchronisations and graph replays per region so tests can put a
    budget on them (e.g. "a decode step is one graph replay and zero synchronisations")."""

    def __init__(self):
        self.counters: Counter = Counter()
        self.regions: Dict[str, Counter] = {}
        self._stack: List[str] = []

    def _bump(self, key: str, n: int = 1) -> None:
        if not LAUNCH_TRACE_ON:
            return
        self.counters[key] += n
        for r in self._stack:
            self.regions.setdefault(r, Counter())[key] += n

    def record_kernel(self, name: str = "", n: int = 1) -> None:
        self._bump("kernels", n)
        if name:
            self._bump(f"kernel:{name}", n)

    def record_copy(self, direction: str, nbytes: int) -> None:
        self._bump(f"copies_{direction}")
        self._bump(f"bytes_{direction}", nbytes)

    def record_wait(self) -> None:
        self._bump("waits")

    def record_commit(self) -> None:
        self._bump("graph_replays")

    @contextlib.contextmanager
    def trace_region(self, name: str):
        from .. import ops
        k0 = ops.launch_count()
        self._stack.append(name)
        try:
            yield
        finally:
            self._stack.pop()
            if LAUNCH_TRACE_ON:
                d = ops.launch_count() - k0
                self.regions.setdefault(name, Counter())["kernels"] += d
                self.counters["kernels"] += d if not self._stack else 0

    def write_json(self, path: str) -> None:
        with open(path, "w") as f:
            json.dump({"counters": dict(self.counters), "regions": {k: dict(v) for k, v in self.regions.items()}}, f, indent=1)

    def reset(self) -> None:
        self.counters.clear()
        self.regions.clear()


launch_tracer = LaunchTracer()
