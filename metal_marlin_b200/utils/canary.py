"""Canary-padded buffers: the stand-in for a memory checker where none can be run.  A guarded tensor sits in the middle of a
larger allocation whose margins are filled with a byte pattern; after the kernels under test have written their output the
margins are compared with the pattern, so a store outside the tensor (an off-by-one tile edge, a missing row guard, a
stride mix-up) is caught at the test that caused it instead of corrupting a neighbour.

    with CanaryArena(device) as arena:
        out = arena.empty((37, 2048), torch.bfloat16)
        ops.linear(x, w, out=out)
    # leaving the block checks every margin; arena.check() can also be called at any point

``guard_outputs()`` patches ``torch.empty`` / ``torch.zeros`` / ``torch.empty_like`` for the duration of a block so that every
buffer an op allocates for its result is guarded, without touching the op.

Parity: reference ``metal_marlin/utils/buffer_guard.py`` / the debug-build bounds checks of its Metal dispatch layer
(``metal_dispatch.py`` validation mode).
"""
from __future__ import annotations

import contextlib
from typing import List, Tuple

import torch

PATTERN = 0xA5
DEFAULT_MARGIN = 512          # bytes on each side


class CanaryViolation(RuntimeError):
    pass


class CanaryArena:
    def __init__(self, device="cuda", margin: int = DEFAULT_MARGIN):
        self.device, self.margin = torch.device(device), int(margin)
        self._blocks: List[Tuple[torch.Tensor, int, int, str]] = []      # raw bytes, payload offset, payload bytes, label

    def empty(self, shape, dtype=torch.bfloat16, label: str = "") -> torch.Tensor:
        if isinstance(shape, int):
            shape = (shape,)
        n = 1
        for s in shape:
            n *= int(s)
        es = torch.empty(0, dtype=dtype).element_size()
        nbytes = n * es
        m = (self.margin + 255) // 256 * 256                    # keeps the payload 256-byte aligned like a fresh allocation
        raw = torch.full((m + nbytes + m,), PATTERN, dtype=torch.uint8, device=self.device)
        self._blocks.append((raw, m, nbytes, label or f"buffer {len(self._blocks)} {tuple(shape)}"))
        return raw[m: m + nbytes].view(dtype).view(*shape)

    def zeros(self, shape, dtype=torch.bfloat16, label: str = "") -> torch.Tensor:
        t = self.empty(shape, dtype, label)
        t.zero_()
        return t

    def check(self) -> None:
        """Raises :class:`CanaryViolation` naming the first buffer whose margin changed (and where)."""
        for raw, off, nbytes, label in self._blocks:
            for side, seg, base in (("before", raw[:off], -off), ("after", raw[off + nbytes:], nbytes)):
                bad = (seg != PATTERN).nonzero()
                if bad.numel():
                    first = int(bad[0])
                    raise CanaryViolation(f"{label}: {int(bad.numel())} byte(s) written {side} the buffer, first at offset "
                                          f"{base + first:+d} relative to its {'start' if side == 'before' else 'start (size ' + str(nbytes) + ')'}")

    def __enter__(self):
        return self

    def __exit__(self, et, ev, tb):
        if et is None:
            if self.device.type == "cuda":
                torch.cuda.synchronize(self.device)
            self.check()
        return False


@contextlib.contextmanager
def guard_outputs(device="cuda", margin: int = DEFAULT_MARGIN):
    """Every ``torch.empty`` / ``torch.zeros`` / ``torch.empty_like`` / ``torch.zeros_like`` on ``device`` inside the block
    returns a guarded buffer; the margins are checked when the block ends."""
    dev = torch.device(device)
    arena = CanaryArena(dev, margin)
    o_empty, o_zeros, o_empty_like, o_zeros_like = torch.empty, torch.zeros, torch.empty_like, torch.zeros_like

    def on_dev(kw):
        d = kw.get("device")
        return d is not None and torch.device(d).type == dev.type and kw.get("pin_memory") in (None, False)

    def _shape(a):
        return tuple(a[0]) if len(a) == 1 and isinstance(a[0], (tuple, list, torch.Size)) else tuple(a)

    def empty(*a, **kw):
        if not on_dev(kw) or kw.get("dtype") in (torch.bool,) or kw.get("memory_format") is not None:
            return o_empty(*a, **kw)
        return arena.empty(_shape(a), kw.get("dtype") or torch.get_default_dtype())

    def zeros(*a, **kw):
        if not on_dev(kw) or kw.get("dtype") in (torch.bool,):
            return o_zeros(*a, **kw)
        return arena.zeros(_shape(a), kw.get("dtype") or torch.get_default_dtype())

    def empty_like(t, **kw):
        if t.device.type != dev.type or kw or not t.is_contiguous() or t.dtype == torch.bool:
            return o_empty_like(t, **kw)
        return arena.empty(tuple(t.shape), t.dtype)

    def zeros_like(t, **kw):
        if t.device.type != dev.type or kw or not t.is_contiguous() or t.dtype == torch.bool:
            return o_zeros_like(t, **kw)
        return arena.zeros(tuple(t.shape), t.dtype)

    torch.empty, torch.zeros, torch.empty_like, torch.zeros_like = empty, zeros, empty_like, zeros_like
    try:
        yield arena
    finally:
        torch.empty, torch.zeros, torch.empty_like, torch.zeros_like = o_empty, o_zeros, o_empty_like, o_zeros_like
    if dev.type == "cuda":
        torch.cuda.synchronize(dev)
    arena.check()
