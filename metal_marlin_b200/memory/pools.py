"""Recycling pools for transient device buffers and a transfer stream.

``BufferPool`` keeps released tensors in three size tiers and serves later requests best-fit from the matching tier
(bounded by a byte limit with least-recently-used eviction and an idle time-out); ``TransferStream`` moves a dictionary
of host tensors to the device on a side stream through pinned staging and hands back an event to wait on;
``RingBuffer`` is the step-scoped bump allocator under its reference name, with a per-device instance.

Parity: reference ``metal_marlin/memory/buffer_pool.py`` (``BufferPool`` ``:80``: tiers, best fit ``:146``, ``acquire`` ``:176``,
``release`` ``:214``, eviction ``:263``, ``cleanup_old_buffers`` ``:309``, stats), ``memory/buffer_recycler.py``,
``memory/transfer_stream.py`` (``TransferStream.transfer_async`` ``:39``), ``buffer_ring.py`` (``RingBuffer`` ``:61``,
``get_ring_buffer`` ``:219``).  Allocation of long-lived state goes through ``Arena`` (one slab, native bookkeeping); this pool
is for code that asks for scratch tensors of recurring sizes outside a captured graph.
"""
from __future__ import annotations

import threading
import time
from collections import OrderedDict
from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch

from .arena import BumpAllocator
from .streaming import PinnedPool

SMALL_MAX = 1 << 20          # tier bounds in bytes
MEDIUM_MAX = 64 << 20


@dataclass
class BufferPoolStats:
    hits: int = 0
    misses: int = 0
    evictions: int = 0
    bytes_pooled: int = 0
    bytes_in_use: int = 0
    peak_bytes: int = 0

    @property
    def hit_rate(self) -> float:
        n = self.hits + self.misses
        return self.hits / n if n else 0.0

    def to_dict(self) -> dict:
        return {"hits": self.hits, "misses": self.misses, "evictions": self.evictions, "hit_rate": round(self.hit_rate, 4),
                "bytes_pooled": self.bytes_pooled, "bytes_in_use": self.bytes_in_use, "peak_bytes": self.peak_bytes}


class BufferPool:
    """``acquire(nbytes)`` returns a uint8 tensor of at least ``nbytes`` (view it as needed), ``release`` gives it back."""

    def __init__(self, device="cpu", max_bytes: int = 1 << 30, max_waste: float = 2.0, idle_seconds: float = 60.0):
        self.device = torch.device(device)
        self.max_bytes, self.max_waste, self.idle_seconds = max_bytes, max_waste, idle_seconds
        # per tier: buffers keyed by id, oldest release first
        self._tiers: Dict[str, "OrderedDict[int, Tuple[torch.Tensor, float]]"] = {t: OrderedDict() for t in ("small", "medium", "large")}
        self._lock = threading.Lock()
        self.stats = BufferPoolStats()

    @staticmethod
    def tier_of(nbytes: int) -> str:
        return "small" if nbytes <= SMALL_MAX else ("medium" if nbytes <= MEDIUM_MAX else "large")

    def acquire(self, nbytes: int) -> torch.Tensor:
        with self._lock:
            tier = self._tiers[self.tier_of(nbytes)]
            best = None
            for key, (buf, _t) in tier.items():
                n = buf.numel()
                if nbytes <= n <= nbytes * self.max_waste and (best is None or n < tier[best][0].numel()):
                    best = key
            if best is not None:
                buf, _ = tier.pop(best)
                self.stats.hits += 1
                self.stats.bytes_pooled -= buf.numel()
            else:
                buf = None
                self.stats.misses += 1
        if buf is None:
            buf = torch.empty(max(nbytes, 1), dtype=torch.uint8, device=self.device)
        with self._lock:
            self.stats.bytes_in_use += buf.numel()
            self.stats.peak_bytes = max(self.stats.peak_bytes, self.stats.bytes_in_use + self.stats.bytes_pooled)
        return buf

    def acquire_like(self, shape, dtype=torch.bfloat16) -> torch.Tensor:
        n = 1
        for d in shape:
            n *= int(d)
        nbytes = n * torch.empty(0, dtype=dtype).element_size()
        return self.acquire(nbytes)[:nbytes].view(dtype).view(*shape)

    def release(self, buf: torch.Tensor) -> None:
        base = buf if buf.dtype == torch.uint8 and buf.dim() == 1 and buf._base is None else (buf._base if buf._base is not None else buf)
        base = base.view(torch.uint8).reshape(-1) if base.dtype != torch.uint8 or base.dim() != 1 else base
        n = base.numel()
        with self._lock:
            self.stats.bytes_in_use = max(0, self.stats.bytes_in_use - n)
            if n > self.max_bytes:
                return
            self._evict_to(self.max_bytes - n)
            self._tiers[self.tier_of(n)][id(base)] = (base, time.monotonic())
            self.stats.bytes_pooled += n

    def _evict_to(self, target: int) -> None:
        while self.stats.bytes_pooled > target:
            oldest = min(((t, k, v[1]) for t, d in self._tiers.items() for k, v in d.items()), key=lambda e: e[2], default=None)
            if oldest is None:
                break
            buf, _ = self._tiers[oldest[0]].pop(oldest[1])
            self.stats.bytes_pooled -= buf.numel()
            self.stats.evictions += 1

    def cleanup_old_buffers(self, now: Optional[float] = None) -> int:
        """Drop buffers released more than ``idle_seconds`` ago; returns how many."""
        now = time.monotonic() if now is None else now
        n = 0
        with self._lock:
            for d in self._tiers.values():
                for k in [k for k, (_b, t) in d.items() if now - t > self.idle_seconds]:
                    buf, _ = d.pop(k)
                    self.stats.bytes_pooled -= buf.numel()
                    self.stats.evictions += 1
                    n += 1
        return n

    def clear(self) -> None:
        with self._lock:
            for d in self._tiers.values():
                d.clear()
            self.stats.bytes_pooled = 0

    def get_stats(self) -> dict:
        s = self.stats.to_dict()
        s["buffers"] = {t: len(d) for t, d in self._tiers.items()}
        return s


class TransferStream:
    """Host -> device copies off the compute stream: ``transfer_async`` stages every tensor in pinned memory, issues the
    copies on its own stream and returns ``(device tensors, event)``; consumers call ``wait(event)`` (makes the current stream
    wait) or ``synchronize()``."""

    def __init__(self, device="cuda:0", pool: Optional[PinnedPool] = None):
        self.device = torch.device(device)
        self.cuda = self.device.type == "cuda"
        self.stream = torch.cuda.Stream(self.device) if self.cuda else None
        self.pool = pool or PinnedPool()
        self.bytes_moved = 0
        self._staged = []

    def transfer_async(self, tensors: Dict[str, torch.Tensor]):
        if not self.cuda:
            return {k: v.to(self.device) for k, v in tensors.items()}, None
        out = {}
        with torch.cuda.stream(self.stream):
            for k, v in tensors.items():
                n = v.numel() * v.element_size()
                stage = self.pool.get(n)
                stage[:n].view(v.dtype).view(v.shape).copy_(v)
                out[k] = stage[:n].view(v.dtype).view(v.shape).to(self.device, non_blocking=True)
                self._staged.append(stage)
                self.bytes_moved += n
            ev = torch.cuda.Event()
            ev.record(self.stream)
        return out, ev

    def wait(self, event) -> None:
        if event is not None:
            torch.cuda.current_stream(self.device).wait_event(event)

    def synchronize(self) -> None:
        if self.cuda:
            self.stream.synchronize()
        for s in self._staged:
            self.pool.put(s)
        self._staged.clear()


class RingBuffer(BumpAllocator):
    """Step-scoped transient allocations (``alloc`` advances an offset, ``reset`` starts over) under the reference's name."""

    def __init__(self, device="cpu", capacity: int = 256 << 20, alignment: int = 128):
        super().__init__(capacity, device, alignment)

    capacity = property(lambda self: self.slab.numel())
    used = property(lambda self: self.cursor)
    available = property(lambda self: self.slab.numel() - self.cursor)
    high_water_mark = property(lambda self: self.high_water)

    def can_alloc(self, nbytes: int) -> bool:
        start = (self.cursor + self.alignment - 1) // self.alignment * self.alignment
        return start + nbytes <= self.slab.numel()

    def stats(self) -> dict:
        return {"capacity": self.capacity, "used": self.used, "available": self.available, "high_water_mark": self.high_water_mark}


_rings: Dict[str, RingBuffer] = {}


def get_ring_buffer(device="cpu", capacity: int = 256 << 20) -> RingBuffer:
    key = str(torch.device(device))
    if key not in _rings:
        _rings[key] = RingBuffer(device, capacity)
    return _rings[key]


def reset_ring_buffer(device="cpu") -> None:
    r = _rings.get(str(torch.device(device)))
    if r is not None:
        r.reset()


# ------------------------------------------------------------------------------------------------ transient (per-pass) buffer
class TransientBuffer:
    """Per-pass scratch over one slab: ``allocate(size) -> (slab, offset)`` (256-byte aligned), ``tensor(shape, dtype)`` for a view,
    ``reset()`` in O(1) at the start of a pass; one shared instance per device through ``get_for_device``.  Reference
    ``transient_buffer_cpp.py:59`` (``TransientBufferCPP``: ``allocate`` / ``allocate_bytes`` / ``reset`` / ``capacity`` / ``used`` / ``available`` /
    ``utilization`` / ``stats`` / ``get_for_device`` / ``reset_global``)."""
    _instances: dict = {}

    def __init__(self, device=None, capacity: int = 100 * 1024 * 1024):
        from .arena import BumpAllocator
        dev = torch.device(device) if device is not None else torch.device("cuda" if torch.cuda.is_available() else "cpu")
        self._bump = BumpAllocator(int(capacity), dev)
        self._device, self._resets, self._allocs = dev, 0, 0

    def reset(self) -> None:
        self._bump.reset()
        self._resets += 1

    def allocate(self, size: int):
        t = self._bump.alloc((int(size),), torch.uint8)
        self._allocs += 1
        return self._bump.slab, t.data_ptr() - self._bump.slab.data_ptr()

    allocate_bytes = allocate

    def tensor(self, shape, dtype=torch.bfloat16) -> torch.Tensor:
        self._allocs += 1
        return self._bump.alloc(tuple(shape), dtype)

    @property
    def capacity(self) -> int:
        return self._bump.slab.numel()

    @property
    def used(self) -> int:
        return self._bump.cursor

    @property
    def available(self) -> int:
        return self.capacity - self.used

    @property
    def utilization(self) -> float:
        return self.used / self.capacity if self.capacity else 0.0

    @property
    def is_cpp_backend(self) -> bool:
        return False                         # a cursor over one tensor: there is nothing for native code to add

    def stats(self) -> dict:
        return {"capacity": self.capacity, "used": self.used, "available": self.available, "utilization": self.utilization,
                "high_water": self._bump.high_water, "allocations": self._allocs, "resets": self._resets, "device": str(self._device)}

    @classmethod
    def get_for_device(cls, device=None, capacity: int = 100 * 1024 * 1024) -> "TransientBuffer":
        key = str(torch.device(device) if device is not None else torch.device("cuda" if torch.cuda.is_available() else "cpu"))
        inst = cls._instances.get(key)
        if inst is None or inst.capacity < capacity:
            inst = cls._instances[key] = cls(key, capacity)
        return inst

    @classmethod
    def reset_global(cls) -> None:
        cls._instances.clear()

    @classmethod
    def is_available(cls) -> bool:
        return True


TransientBufferCPP = TransientBuffer


def get_transient_buffer_cpp(device=None, capacity: int = 100 * 1024 * 1024) -> TransientBuffer:
    return TransientBuffer.get_for_device(device, capacity)


def reset_transient_buffer_cpp() -> None:
    TransientBuffer.reset_global()


def transient_buffer_cpp_stats(device=None):
    key = str(torch.device(device) if device is not None else torch.device("cuda" if torch.cuda.is_available() else "cpu"))
    inst = TransientBuffer._instances.get(key)
    return inst.stats() if inst is not None else None
