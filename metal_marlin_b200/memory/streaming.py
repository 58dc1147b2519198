"""Pinned staging pool and asynchronous weight streaming (host -> device on a copy stream, double buffered)."""
from __future__ import annotations

import threading
from collections import deque
from typing import Callable, Deque, Dict, Iterable, Iterator, List, Optional, Sequence, Tuple

import torch


class PinnedPool:
    """Recycles pinned host buffers by size class (powers of two) so repeated transfers never re-pin memory."""

    def __init__(self, max_bytes: int = 1 << 30):
        self.max_bytes, self.held = max_bytes, 0
        self._free: Dict[int, List[torch.Tensor]] = {}
        self._lock = threading.Lock()
        self.hits = self.misses = 0

    @staticmethod
    def _cls(n: int) -> int:
        return 1 << max(12, (n - 1).bit_length())

    def get(self, nbytes: int) -> torch.Tensor:
        c = self._cls(nbytes)
        with self._lock:
            lst = self._free.get(c)
            if lst:
                self.hits += 1
                self.held -= c
                return lst.pop()
            self.misses += 1
        return torch.empty(c, dtype=torch.uint8, pin_memory=torch.cuda.is_available())

    def put(self, buf: torch.Tensor) -> None:
        c = buf.numel()
        with self._lock:
            if self.held + c <= self.max_bytes:
                self._free.setdefault(c, []).append(buf)
                self.held += c


class WeightStreamer:
    """Streams a sequence of named host tensors to the device ahead of use: while layer ``i`` computes, layer
    ``i + depth`` is copied on a side stream from pinned staging buffers (models larger than HBM, expert offload)."""

    def __init__(self, device, depth: int = 2, pool: Optional[PinnedPool] = None):
        self.device = torch.device(device)
        self.depth = depth
        self.pool = pool or PinnedPool()
        self.cuda = self.device.type == "cuda"
        self.stream = torch.cuda.Stream(self.device) if self.cuda else None
        self.bytes_streamed = 0

    def _issue(self, tensors: Dict[str, torch.Tensor]):
        out, staged, ev = {}, [], None
        if not self.cuda:
            return {k: v.to(self.device) for k, v in tensors.items()}, staged, ev
        with torch.cuda.stream(self.stream):
            for k, v in tensors.items():
                v = v.contiguous()
                n = v.numel() * v.element_size()
                st = self.pool.get(n)
                st[:n].copy_(v.view(torch.uint8).reshape(-1))
                d = torch.empty(n, dtype=torch.uint8, device=self.device)
                d.copy_(st[:n], non_blocking=True)
                out[k] = d.view(v.dtype).view(v.shape)
                staged.append(st)
                self.bytes_streamed += n
            ev = torch.cuda.Event()
            ev.record(self.stream)
        return out, staged, ev

    def stream_layers(self, layers: Iterable[Dict[str, torch.Tensor]]) -> Iterator[Dict[str, torch.Tensor]]:
        """Yields device copies of each layer's tensors in order, keeping ``depth`` layers in flight."""
        it = iter(layers)
        q: Deque = deque()
        for _ in range(self.depth):
            nxt = next(it, None)
            if nxt is None:
                break
            q.append(self._issue(nxt))
        while q:
            out, staged, ev = q.popleft()
            if ev is not None:
                torch.cuda.current_stream(self.device).wait_event(ev)
            nxt = next(it, None)
            if nxt is not None:
                q.append(self._issue(nxt))
            yield out
            for st in staged:
                self.pool.put(st)
