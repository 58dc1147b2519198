"""Host and device memory queries, tensor-size estimates, batch sizing and padding helpers.  Parity: reference
``metal_marlin/utils/memory.py`` (``MemoryInfo`` ``:37``, ``get_system_memory`` ``:57``, ``estimate_tensor_memory`` ``:264``,
``compute_optimal_batch_size`` ``:289``, ``should_reduce_allocation`` ``:367``), ``utils/padding.py`` (``round_up``, ``pad_numpy_2d``,
``pad_torch_2d``) and ``utils/prefetch.py`` (``SystemMemoryInfo``, ``TensorMetadata``, ``AdaptivePrefetcher``)."""
from __future__ import annotations

import os
import threading
from dataclasses import dataclass
from typing import Any, Dict, Iterator, List, Optional, Sequence, Tuple

import numpy as np
import torch

_GB = float(1 << 30)


@dataclass
class MemoryInfo:
    total_ram_gb: float
    available_ram_gb: float
    gpu_total_gb: float
    gpu_available_gb: float
    is_unified_memory: bool = False


@dataclass
class SystemMemoryInfo:
    total_ram_gb: float
    available_ram_gb: float
    used_ram_gb: float
    swap_total_gb: float
    swap_used_gb: float


def _meminfo() -> Dict[str, float]:
    out = {}
    try:
        with open("/proc/meminfo") as f:
            for line in f:
                k, v = line.split(":", 1)
                out[k] = float(v.split()[0]) * 1024
    except OSError:
        import psutil
        vm, sw = psutil.virtual_memory(), psutil.swap_memory()
        out = {"MemTotal": vm.total, "MemAvailable": vm.available, "SwapTotal": sw.total, "SwapFree": sw.free}
    return out


def get_system_memory(*, refresh: bool = False) -> MemoryInfo:
    m = _meminfo()
    if torch.cuda.is_available():
        free, total = torch.cuda.mem_get_info()
    else:
        free = total = 0
    return MemoryInfo(m.get("MemTotal", 0) / _GB, m.get("MemAvailable", 0) / _GB, total / _GB, free / _GB, False)


def get_system_memory_detailed() -> SystemMemoryInfo:
    m = _meminfo()
    tot, av = m.get("MemTotal", 0), m.get("MemAvailable", 0)
    return SystemMemoryInfo(tot / _GB, av / _GB, (tot - av) / _GB, m.get("SwapTotal", 0) / _GB,
                            (m.get("SwapTotal", 0) - m.get("SwapFree", 0)) / _GB)


def get_metal_memory_pressure() -> str:
    """``normal`` / ``warn`` / ``critical`` from the device's free memory (kept under the reference's name)."""
    from ..memory.pressure import MemoryPressureMonitor, PressureLevel
    lvl = MemoryPressureMonitor().check()
    return {PressureLevel.NORMAL: "normal", PressureLevel.WARNING: "warn", PressureLevel.CRITICAL: "critical"}[lvl]


def should_reduce_allocation(threshold: str = "warn") -> bool:
    p = get_metal_memory_pressure()
    return p == "critical" or (threshold == "warn" and p == "warn")


def _itemsize(dtype) -> int:
    if isinstance(dtype, torch.dtype):
        return torch.empty(0, dtype=dtype).element_size()
    if isinstance(dtype, str) and dtype in ("bf16", "bfloat16"):
        return 2
    return int(np.dtype(dtype).itemsize)


def estimate_tensor_memory(shape: Tuple[int, ...], dtype=np.float16) -> int:
    n = 1
    for d in shape:
        n *= int(d)
    return n * _itemsize(dtype)


def compute_optimal_batch_size(tensor_shapes: Sequence[Tuple[int, ...]], available_memory_gb: float, dtype=np.float16,
                               safety_factor: float = 0.7) -> int:
    """Largest batch whose per-sample tensors (``tensor_shapes`` are one sample's) fit ``safety_factor`` of the memory; >= 1."""
    per = sum(estimate_tensor_memory(s, dtype) for s in tensor_shapes)
    if per <= 0:
        return 1
    return max(1, int(available_memory_gb * _GB * safety_factor // per))


def round_up(value: int, multiple: int) -> int:
    if multiple <= 0:
        raise ValueError("multiple must be positive")
    return ((value + multiple - 1) // multiple) * multiple


def pad_numpy_2d(array: np.ndarray, *, rows_multiple: int, cols_multiple: int, value: float = 0.0):
    r, c = array.shape
    R, C = round_up(r, rows_multiple), round_up(c, cols_multiple)
    if (R, C) == (r, c):
        return array, (r, c)
    out = np.full((R, C), value, dtype=array.dtype)
    out[:r, :c] = array
    return out, (r, c)


def pad_torch_2d(tensor: torch.Tensor, *, rows_multiple: int, cols_multiple: int, value: float = 0.0):
    r, c = tensor.shape
    R, C = round_up(r, rows_multiple), round_up(c, cols_multiple)
    if (R, C) == (r, c):
        return tensor, (r, c)
    return torch.nn.functional.pad(tensor, (0, C - c, 0, R - r), value=value), (r, c)


@dataclass
class TensorMetadata:
    name: str
    file_path: str
    dtype: str
    shape: Tuple[int, ...]
    nbytes: int


class AdaptivePrefetcher:
    """Iterates the tensors of safetensors files in batches that fit a memory budget; while one batch is being used the
    next one is read by a background thread."""

    def __init__(self, files: Sequence[str], budget_bytes: Optional[int] = None, memory_fraction: float = 0.25):
        from ..formats.safetensors_io import SafetensorsFile
        self.meta: List[TensorMetadata] = []
        for fp in files:
            with SafetensorsFile(fp) as sf:
                for k in sf.keys():
                    shp = tuple(sf.shape(k))
                    info = sf.info(k)
                    nb = int(info["data_offsets"][1] - info["data_offsets"][0]) if "data_offsets" in info else 0
                    self.meta.append(TensorMetadata(k, fp, sf.dtype_str(k), shp, nb))
        if budget_bytes is None:
            budget_bytes = int(get_system_memory().available_ram_gb * _GB * memory_fraction)
        self.budget = max(1, budget_bytes)

    def batches(self) -> List[List[TensorMetadata]]:
        out, cur, size = [], [], 0
        for m in self.meta:
            if cur and size + m.nbytes > self.budget:
                out.append(cur)
                cur, size = [], 0
            cur.append(m)
            size += m.nbytes
        if cur:
            out.append(cur)
        return out

    def _load(self, batch: List[TensorMetadata]) -> Dict[str, torch.Tensor]:
        from ..formats.safetensors_io import SafetensorsFile
        res: Dict[str, torch.Tensor] = {}
        by_file: Dict[str, List[str]] = {}
        for m in batch:
            by_file.setdefault(m.file_path, []).append(m.name)
        for fp, names in by_file.items():
            with SafetensorsFile(fp) as sf:
                for n in names:
                    res[n] = sf.get_tensor(n)
        return res

    def __iter__(self) -> Iterator[Dict[str, torch.Tensor]]:
        bs = self.batches()
        nxt: Dict[str, Any] = {}

        def work(i):
            nxt["v"] = self._load(bs[i])
        th = None
        if bs:
            th = threading.Thread(target=work, args=(0,))
            th.start()
        for i in range(len(bs)):
            th.join()
            cur = nxt.pop("v")
            if i + 1 < len(bs):
                th = threading.Thread(target=work, args=(i + 1,))
                th.start()
            yield cur


def pad_to_multiple(tensor, dim: int, multiple: int = 8):
    """Zero-pad ``tensor`` along ``dim`` up to the next multiple: ``(padded, pad_size)`` (the tensor itself and 0 when it fits)."""
    import torch
    if multiple <= 0:
        raise ValueError(f"multiple must be > 0, got {multiple}")
    d = dim % tensor.dim()
    pad = (-tensor.size(d)) % multiple
    if pad == 0:
        return tensor, 0
    shape = list(tensor.shape)
    shape[d] = pad
    return torch.cat([tensor, torch.zeros(shape, dtype=tensor.dtype, device=tensor.device)], d), pad


def unpad(tensor, dim: int, pad_size: int):
    """Undo :func:`pad_to_multiple`."""
    if pad_size == 0:
        return tensor
    d = dim % tensor.dim()
    return tensor.narrow(d, 0, tensor.size(d) - pad_size)
