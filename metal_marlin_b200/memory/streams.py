"""Stream and event pools, and device / interconnect discovery.

The engine runs its decode step on one stream (captured into CUDA graphs); copies (weight streaming, KV swaps, prompt
cache promotion) and collectives get their own streams so they overlap compute.  ``StreamPool`` hands out named,
prioritised streams per device; ``EventPool`` recycles CUDA events and offers a bounded wait (``AsyncEvent``);
``discover_devices`` reports what the scheduler and the mesh builder need: SM count, memory, peer access, NVLink links
(through NVML when it is importable) and whether NVLS-style multicast is plausible (all pairs peer-accessible).
Everything degrades to empty results on a machine without CUDA.

Parity: reference ``metal_marlin/cpp/src/device.cpp`` / ``device_discovery.cpp`` (device properties, queue creation:
primary / decode / transfer), ``events.mm`` (``AsyncEvent`` wait with timeout) and ``encoder_cache.mm`` (per-thread reuse of
submission objects), re-thought for CUDA streams and events.
"""
from __future__ import annotations

import threading
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

ROLES = ("compute", "decode", "copy", "comm")
_PRIORITY = {"compute": 0, "decode": -1, "copy": 0, "comm": -1}      # lower number = higher priority


class StreamPool:
    """Named streams per device; the same (device, role, index) always returns the same stream."""

    def __init__(self):
        self._streams: Dict[tuple, "torch.cuda.Stream"] = {}
        self._lock = threading.Lock()

    def get(self, role: str = "compute", device: Optional[int] = None, index: int = 0):
        if role not in ROLES:
            raise ValueError(f"unknown stream role {role!r}; expected one of {ROLES}")
        if not torch.cuda.is_available():
            return None
        dev = torch.cuda.current_device() if device is None else int(device)
        key = (dev, role, index)
        with self._lock:
            s = self._streams.get(key)
            if s is None:
                s = torch.cuda.Stream(device=dev, priority=_PRIORITY[role])
                self._streams[key] = s
            return s

    def synchronize(self, device: Optional[int] = None) -> None:
        for (dev, _, _), s in list(self._streams.items()):
            if device is None or dev == device:
                s.synchronize()

    def __len__(self) -> int:
        return len(self._streams)


class AsyncEvent:
    """A recorded point of a stream that can be polled or waited for with a deadline (no unbounded host waits)."""

    def __init__(self, event=None):
        self.event = event
        self._done = event is None

    def query(self) -> bool:
        if not self._done:
            self._done = bool(self.event.query())
        return self._done

    def wait(self, timeout_s: float = 10.0, poll_s: float = 50e-6) -> bool:
        t0 = time.monotonic()
        while not self.query():
            if time.monotonic() - t0 > timeout_s:
                return False
            time.sleep(poll_s)
        return True


class EventPool:
    def __init__(self, timing: bool = False):
        self.timing = timing
        self._free: List = []
        self.created = 0
        self.reused = 0

    def record(self, stream=None) -> AsyncEvent:
        if not torch.cuda.is_available():
            return AsyncEvent(None)
        if self._free:
            ev = self._free.pop()
            self.reused += 1
        else:
            ev = torch.cuda.Event(enable_timing=self.timing)
            self.created += 1
        ev.record(stream if stream is not None else torch.cuda.current_stream())
        return AsyncEvent(ev)

    def release(self, ae: AsyncEvent) -> None:
        if ae.event is not None:
            self._free.append(ae.event)
            ae.event = None
            ae._done = True


@dataclass
class DeviceInfo:
    index: int
    name: str
    sm_count: int
    total_memory: int
    capability: tuple
    peers: List[int] = field(default_factory=list)          # devices this one can address directly
    nvlink_links: Optional[int] = None                      # active NVLink links (NVML), None if unknown


def _nvml_links(index: int, nvml=None) -> Optional[int]:
    try:
        if nvml is None:
            import pynvml as nvml       # type: ignore
            nvml.nvmlInit()
        h = nvml.nvmlDeviceGetHandleByIndex(index)
        n = 0
        for link in range(18):
            try:
                if nvml.nvmlDeviceGetNvLinkState(h, link):
                    n += 1
            except Exception:
                break
        return n
    except Exception:
        return None


def discover_devices(nvml=None) -> List[DeviceInfo]:
    """One entry per visible CUDA device (empty without CUDA).  ``nvml``: an NVML-like module (tests pass a fake)."""
    if not torch.cuda.is_available():
        return []
    out = []
    n = torch.cuda.device_count()
    for i in range(n):
        p = torch.cuda.get_device_properties(i)
        peers = [j for j in range(n) if j != i and torch.cuda.can_device_access_peer(i, j)]
        out.append(DeviceInfo(i, p.name, p.multi_processor_count, p.total_memory, (p.major, p.minor), peers, _nvml_links(i, nvml)))
    return out


def multicast_plausible(devs: List[DeviceInfo]) -> bool:
    """NVSwitch-style multicast needs every device to reach every other one directly."""
    n = len(devs)
    return n > 1 and all(len(d.peers) == n - 1 for d in devs)


_default_streams = StreamPool()


def get_stream(role: str = "compute", device: Optional[int] = None, index: int = 0):
    return _default_streams.get(role, device, index)
