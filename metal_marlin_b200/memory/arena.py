"""Sub-allocating arena over one slab tensor, bump allocator for step-scoped scratch, named workspace buffers."""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .. import _build

_ELT = {torch.float32: 4, torch.float16: 2, torch.bfloat16: 2, torch.int32: 4, torch.int64: 8, torch.uint8: 1, torch.int8: 1,
        torch.float64: 8, torch.bool: 1, torch.int16: 2}


def _native():
    _build.load(require=True)
    return torch.ops.mmb200


class Arena:
    """Best-fit allocator with coalescing, pin / unpin and priority + LRU eviction over ``slab`` (a uint8 tensor on any
    device; for the symmetric heap pass the peer-mapped buffer).  ``alloc`` returns a typed view; the view's offset is
    its handle."""

    def __init__(self, capacity_bytes: int = 0, device="cpu", alignment: int = 256, slab: Optional[torch.Tensor] = None,
                 pin_memory: bool = False):
        if slab is None:
            slab = torch.empty(capacity_bytes, dtype=torch.uint8, device=device, pin_memory=pin_memory and str(device) == "cpu")
        assert slab.dtype == torch.uint8 and slab.is_contiguous()
        self.slab = slab
        self.alignment = alignment
        self._h = _native().arena_create(slab.numel(), alignment)
        self._live: Dict[int, Tuple[int, str]] = {}          # offset -> (nbytes, tag)
        self.on_evict = None                                  # callable(offset, tag)

    def alloc(self, shape: Sequence[int], dtype=torch.bfloat16, priority: int = 0, allow_evict: bool = False, tag: str = "") -> torch.Tensor:
        n = int(math.prod(shape)) * _ELT[dtype]
        res = list(_native().arena_alloc(self._h, n, priority, allow_evict))
        off, evicted = res[0], res[1:]
        for e in evicted:
            _, t = self._live.pop(e, (0, ""))
            if self.on_evict is not None:
                self.on_evict(e, t)
        if off < 0:
            raise MemoryError(f"arena out of memory: {n} bytes requested, stats {self.stats()}")
        self._live[off] = (n, tag)
        return self.slab[off: off + n].view(dtype).view(*shape)

    def offset_of(self, t: torch.Tensor) -> int:
        return t.data_ptr() - self.slab.data_ptr()

    def free(self, t_or_offset) -> None:
        off = t_or_offset if isinstance(t_or_offset, int) else self.offset_of(t_or_offset)
        _native().arena_free(self._h, off)
        self._live.pop(off, None)

    def pin(self, t: torch.Tensor, pinned: bool = True) -> None:
        _native().arena_pin(self._h, self.offset_of(t), pinned)

    def touch(self, t: torch.Tensor) -> None:
        _native().arena_touch(self._h, self.offset_of(t))

    def compact(self) -> Dict[int, int]:
        """Close the holes between live blocks (pinned blocks stay in place).  The bytes are moved inside the slab; views
        handed out earlier for moved blocks are stale afterwards, the returned ``{old offset: new offset}`` map tells the
        owner where each block went (``view_at`` gives a fresh view)."""
        moves = list(_native().arena_compact(self._h))
        remap: Dict[int, int] = {}
        for i in range(0, len(moves), 3):
            old, new, size = moves[i], moves[i + 1], moves[i + 2]
            if new + size <= old:
                self.slab[new: new + size].copy_(self.slab[old: old + size])
            else:                                   # overlapping slide to lower addresses: go through a temporary
                self.slab[new: new + size].copy_(self.slab[old: old + size].clone())
            remap[old] = new
        self._live = {remap.get(off, off): v for off, v in self._live.items()}
        return remap

    def view_at(self, offset: int, shape: Sequence[int], dtype=torch.bfloat16) -> torch.Tensor:
        n = int(math.prod(shape)) * _ELT[dtype]
        return self.slab[offset: offset + n].view(dtype).view(*shape)

    def stats(self) -> Dict[str, float]:
        cap, used, peak, n_alloc, n_evict, n_blocks, largest, frag = _native().arena_stats(self._h)
        return {"capacity": cap, "used": used, "peak": peak, "allocs": n_alloc, "evictions": n_evict, "blocks": n_blocks,
                "largest_free": largest, "fragmentation": frag / 1e6}

    def close(self) -> None:
        if self._h is not None:
            _native().arena_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class BumpAllocator:
    """Step-scoped scratch: allocations advance a cursor, ``reset()`` frees everything in O(1) (the transient ring of
    the reference).  ``mark`` / ``release`` give nested scopes."""

    def __init__(self, capacity_bytes: int, device="cpu", alignment: int = 256):
        self.slab = torch.empty(capacity_bytes, dtype=torch.uint8, device=device)
        self.alignment, self.cursor, self.high_water = alignment, 0, 0

    def alloc(self, shape: Sequence[int], dtype=torch.bfloat16) -> torch.Tensor:
        n = int(math.prod(shape)) * _ELT[dtype]
        start = (self.cursor + self.alignment - 1) // self.alignment * self.alignment
        if start + n > self.slab.numel():
            raise MemoryError(f"bump allocator exhausted: need {n} bytes at {start} of {self.slab.numel()}")
        self.cursor = start + n
        self.high_water = max(self.high_water, self.cursor)
        return self.slab[start: start + n].view(dtype).view(*shape)

    def mark(self) -> int:
        return self.cursor

    def release(self, mark: int) -> None:
        assert mark <= self.cursor
        self.cursor = mark

    def reset(self) -> None:
        self.cursor = 0


class WorkspaceBuffer:
    """Named persistent buffers that only ever grow (decode state, split-KV partials, logits)."""

    def __init__(self, device="cpu"):
        self.device = device
        self._bufs: Dict[str, torch.Tensor] = {}

    def get(self, name: str, shape: Sequence[int], dtype=torch.bfloat16) -> torch.Tensor:
        n = int(math.prod(shape))
        b = self._bufs.get(name)
        if b is None or b.numel() < n or b.dtype != dtype:
            b = torch.empty(max(n, 1), dtype=dtype, device=self.device)
            self._bufs[name] = b
        return b[:n].view(*shape)

    def nbytes(self) -> int:
        return sum(b.numel() * b.element_size() for b in self._bufs.values())
