"""Feature flags and canonical numeric tables.

Parity: reference ``metal_marlin/_compat.py:60`` (``_init_flags``) and ``:314``
(``get_e2m1_torch_table``).  The reference probes for MPS / PyObjC; this build
probes for CUDA on Blackwell (sm_100) and for the in-tree native extension.
"""
from __future__ import annotations

import functools
import os

import numpy as np
import torch

HAS_TORCH = True
HAS_CUDA = torch.cuda.is_available()
# The reference exposes these names; on this platform they are always False.
HAS_MPS = False
HAS_PYOBJC_METAL = False

# E2M1 code -> value.  Code bit 3 is the sign, bits 2..1 the exponent, bit 0 the mantissa.
E2M1_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0,
               -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0)
E2M1_MAX = 6.0

# NF4 (QLoRA) code book, 16 quantiles of N(0,1) normalised to [-1, 1].
NF4_VALUES = (-1.0, -0.6961928009986877, -0.5250730514526367, -0.39491748809814453,
              -0.28444138169288635, -0.18477343022823334, -0.09105003625154495, 0.0,
              0.07958029955625534, 0.16093020141124725, 0.24611230194568634,
              0.33791524171829224, 0.44070982933044434, 0.5626170039176941,
              0.7229568362236023, 1.0)


def is_blackwell() -> bool:
    """True when the current CUDA device is compute capability 10.x."""
    if not HAS_CUDA:
        return False
    major, _ = torch.cuda.get_device_capability()
    return major == 10


@functools.lru_cache(maxsize=None)
def _e2m1_table_cached(device: str, dtype: torch.dtype) -> torch.Tensor:
    return torch.tensor(E2M1_VALUES, dtype=dtype, device=device)


def get_e2m1_torch_table(device="cpu", dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """16-entry E2M1 decode table on ``device``."""
    return _e2m1_table_cached(str(device), dtype)


def get_e2m1_numpy_table(dtype=np.float32) -> np.ndarray:
    return np.asarray(E2M1_VALUES, dtype=dtype)


def to_numpy(x) -> np.ndarray:
    if isinstance(x, np.ndarray):
        return x
    if isinstance(x, torch.Tensor):
        t = x.detach().cpu()
        if t.dtype == torch.bfloat16:
            t = t.float()
        return t.numpy()
    return np.asarray(x)


def to_torch(x, device=None, dtype=None) -> torch.Tensor:
    if isinstance(x, torch.Tensor):
        t = x
    else:
        arr = np.asarray(x)
        if arr.dtype == np.uint32:
            arr = arr.view(np.int32)
        elif arr.dtype == np.uint16:
            arr = arr.view(np.int16)
        t = torch.from_numpy(np.ascontiguousarray(arr))
    if device is not None or dtype is not None:
        t = t.to(device=device, dtype=dtype)
    return t


def env_flag(name: str, default: bool = False) -> bool:
    v = os.environ.get(name)
    if v is None:
        return default
    return v.strip().lower() in ("1", "true", "yes", "on")
