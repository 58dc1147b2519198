"""Memory-pressure monitor: polls free device (or host) memory and calls registered handlers when a threshold is
crossed, so caches shrink before an allocation fails.  Parity: reference ``metal_marlin/memory`` pressure monitor."""
from __future__ import annotations

import enum
import threading
from typing import Callable, List, Optional, Tuple

import torch


class PressureLevel(enum.IntEnum):
    NORMAL = 0
    WARNING = 1
    CRITICAL = 2


class MemoryPressureMonitor:
    def __init__(self, device=None, warning: float = 0.85, critical: float = 0.95, probe: Optional[Callable[[], Tuple[int, int]]] = None):
        """``probe() -> (free_bytes, total_bytes)``; default: ``torch.cuda.mem_get_info`` or ``psutil`` on CPU."""
        self.device, self.warning, self.critical = device, warning, critical
        self.probe = probe or self._default_probe
        self.handlers: List[Callable[[PressureLevel, float], None]] = []
        self.level = PressureLevel.NORMAL
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None

    def _default_probe(self) -> Tuple[int, int]:
        if torch.cuda.is_available():
            return torch.cuda.mem_get_info(self.device)
        import psutil
        vm = psutil.virtual_memory()
        return vm.available, vm.total

    def register(self, handler: Callable[[PressureLevel, float], None]) -> None:
        self.handlers.append(handler)

    def check(self) -> PressureLevel:
        free, total = self.probe()
        used = 1.0 - free / max(total, 1)
        level = PressureLevel.CRITICAL if used >= self.critical else (PressureLevel.WARNING if used >= self.warning else PressureLevel.NORMAL)
        if level != self.level:
            self.level = level
            for h in self.handlers:
                h(level, used)
        return level

    def start(self, interval_s: float = 1.0) -> None:
        def loop():
            while not self._stop.wait(interval_s):
                self.check()
        self._thread = threading.Thread(target=loop, daemon=True)
        self._thread.start()

    def stop(self) -> None:
        self._stop.set()
        if self._thread:
            self._thread.join(timeout=2)
