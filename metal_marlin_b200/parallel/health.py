"""Failure detection for multi-process serving: heartbeats through the rendezvous store, a watchdog that marks silent
ranks dead, and a guard that turns "a peer is gone" into an exception BEFORE the next collective or in-kernel exchange
is launched (so no rank ever waits on the device for a process that no longer exists).

The reference has request / streaming timeouts and scheduler preemption but no rank-level failure handling
(``metal_marlin/serving/engine.py:477,668-690``); multi-GPU serving here needs it because a decode step contains
device-side waits on peers (bounded at one second, ``csrc/tp_comm.cuh``).  Protocol: every rank writes a monotonically
increasing beat to ``hb/<rank>`` from a daemon thread; ``check()`` compares the peers' beats with the values and times
seen at the previous check and raises :class:`PeerFailure` when a peer has not advanced within ``timeout_s``.  A rank
that leaves on purpose calls ``leave()`` (between steps, with nothing in flight), which the others see at once.
"""
from __future__ import annotations

import threading
import time
from typing import Dict, List, Optional

import torch.distributed as dist


class PeerFailure(RuntimeError):
    def __init__(self, ranks: List[int], reason: str):
        super().__init__(f"rank(s) {ranks} {reason}")
        self.ranks, self.reason = ranks, reason


class DeviceWaitExpired(RuntimeError):
    """A bounded device-side wait of a kernel on THIS GPU ran out (no peer is implied): a pipeline barrier of the tensor-core
    GEMM / attention kernels or of the paged decode kernel."""

    def __init__(self, code: int, what: str):
        super().__init__(f"device-side wait expired (status {code}: {what})")
        self.code, self.what = code, what


class ExpertCapacityOverflow(RuntimeError):
    """The expert-parallel receive buffer was too small for the routed rows (status 120): not a peer failure."""

    def __init__(self, code: int = 120):
        super().__init__("expert-parallel receive buffer overflowed; rows were dropped (status 120)")
        self.code = code


def decode_status(code: int):
    """Meaning of a device status word: ``(kind, ranks, text)`` with kind in
    ``"ok" | "peer" | "local" | "capacity"``.  Only three ranges name a rank: 100-109 tensor-parallel source ``code - 100``,
    121-128 expert-parallel sender ``code - 121``, 140-147 expert-parallel return ``code - 140``."""
    if code == 0:
        return "ok", [], "no wait expired"
    if 100 <= code <= 109:
        return "peer", [code - 100], f"tensor-parallel partial from rank {code - 100} did not arrive"
    if 121 <= code <= 128:
        return "peer", [code - 121], f"expert-parallel rows from rank {code - 121} did not arrive"
    if 140 <= code <= 147:
        return "peer", [code - 140], f"expert-parallel results from rank {code - 140} did not arrive"
    if code == 120:
        return "capacity", [], "expert-parallel receive buffer overflow"
    names = {1: "GEMM producer barrier", 2: "GEMM MMA barrier", 3: "GEMM expansion barrier", 4: "GEMM epilogue barrier",
             42: "attention kernel barrier", 110: "GEMM all-gather tile wait", 200: "paged decode row barrier"}
    return "local", [], names.get(code, "unknown wait")


def raise_for_status(code: int) -> None:
    """Turn a non-zero status word into the matching exception."""
    kind, ranks, text = decode_status(code)
    if kind == "ok":
        return
    if kind == "peer":
        raise PeerFailure(ranks, f"device-side exchange wait expired (status {code}: {text})")
    if kind == "capacity":
        raise ExpertCapacityOverflow(code)
    raise DeviceWaitExpired(code, text)


class Heartbeat:
    def __init__(self, store, rank: int, world: int, interval_s: float = 0.2, timeout_s: float = 2.0, prefix: str = "hb",
                 join_timeout_s: float = 60.0):
        self.store, self.rank, self.world = store, rank, world
        self.interval_s, self.timeout_s, self.prefix = interval_s, timeout_s, prefix
        self.join_timeout_s = join_timeout_s
        self._t0 = time.monotonic()
        self._beat = 0
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._seen: Dict[int, tuple] = {}          # rank -> (beat, time first seen at that value)
        self.store.set(f"{prefix}/{rank}", "0")

    def start(self) -> "Heartbeat":
        def loop():
            while not self._stop.wait(self.interval_s):
                self._beat += 1
                try:
                    self.store.set(f"{self.prefix}/{self.rank}", str(self._beat))
                except Exception:
                    return                          # the store went away with the job
        self._thread = threading.Thread(target=loop, name="mmb200-heartbeat", daemon=True)
        self._thread.start()
        return self

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)

    def leave(self) -> None:
        """Announce an orderly exit (call between steps, with no kernel or collective in flight)."""
        self.stop()
        self.store.set(f"{self.prefix}/{self.rank}", "left")

    def _read(self, r: int) -> Optional[str]:
        """Non-blocking: a blocking ``get`` of a key that does not exist yet would hold the store client and stall this
        rank's own heartbeat thread."""
        key = f"{self.prefix}/{r}"
        try:
            if hasattr(self.store, "check") and not self.store.check([key]):
                return None
            return self.store.get(key).decode()
        except Exception:
            return None

    def dead_ranks(self) -> Dict[int, str]:
        now = time.monotonic()
        dead: Dict[int, str] = {}
        for r in range(self.world):
            if r == self.rank:
                continue
            v = self._read(r)
            if v == "left":
                dead[r] = "left the job"
                continue
            if v is None:
                if now - self._t0 > self.join_timeout_s:
                    dead[r] = "never joined"
                continue
            prev = self._seen.get(r)
            if prev is None or prev[0] != v:
                self._seen[r] = (v, now)
            elif now - prev[1] > self.timeout_s:
                dead[r] = f"sent no heartbeat for {now - prev[1]:.1f} s"
        return dead

    def check(self) -> None:
        """Raise :class:`PeerFailure` when a peer is gone; call before launching a step that waits on peers."""
        dead = self.dead_ranks()
        if dead:
            raise PeerFailure(sorted(dead), "; ".join(f"{r}: {why}" for r, why in sorted(dead.items())))


class StepGuard:
    """Wraps a multi-rank step: checks peer health first, runs the step, then reads the device-side status word of the
    in-kernel exchange and converts a bounded-wait expiry into :class:`PeerFailure`, leaving the CUDA context usable."""

    def __init__(self, heartbeat: Heartbeat, tp_context=None):
        self.hb, self.ctx = heartbeat, tp_context
        self.steps = 0

    def run(self, step_fn):
        self.hb.check()
        out = step_fn()
        self.steps += 1
        if self.ctx is not None:
            raise_for_status(self.ctx.check())
        return out


def make_heartbeat(interval_s: float = 0.2, timeout_s: float = 2.0) -> Heartbeat:
    """Heartbeat over the default process group's store."""
    store = dist.distributed_c10d._get_default_store()
    return Heartbeat(store, dist.get_rank(), dist.get_world_size(), interval_s, timeout_s).start()
