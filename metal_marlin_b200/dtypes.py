"""Dtype configuration: which precision each part of the engine uses.

Parity: reference ``metal_marlin/dtypes.py:65`` (``DTypeConfig`` with weights / activations / accumulation /
scales / kv_cache fields) and its presets at ``metal_marlin/dtypes.py:394-470``.  On B200 the defaults are
bf16 activations (the reference defaults to fp16 on Apple GPUs), fp32 accumulation, fp16 group scales as
stored in the checkpoints, and a bf16 KV cache; fp8 (e4m3) and int8 KV caches are opt-in.
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Dict

import torch

_NAMES: Dict[str, torch.dtype] = {
    "fp32": torch.float32, "float32": torch.float32, "fp16": torch.float16, "float16": torch.float16, "half": torch.float16,
    "bf16": torch.bfloat16, "bfloat16": torch.bfloat16, "fp8": torch.float8_e4m3fn, "fp8_e4m3": torch.float8_e4m3fn,
    "fp8_e5m2": torch.float8_e5m2, "int8": torch.int8, "uint8": torch.uint8,
}
WEIGHT_FORMATS = ("fp4", "int4", "nf4", "int8", "fp8", "int3", "int2", "nf3", "nf2", "trellis", "bf16", "fp16")
KV_FORMATS = ("bf16", "fp16", "fp8", "fp8_e5m2", "int8", "fp4")


def to_torch_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        return name
    try:
        return _NAMES[str(name).lower()]
    except KeyError:
        raise ValueError(f"unknown dtype name {name!r}; known: {sorted(_NAMES)}") from None


@dataclass(frozen=True)
class DTypeConfig:
    weights: str = "fp4"
    activations: str = "bf16"
    accumulation: str = "fp32"
    scales: str = "fp16"
    kv_cache: str = "bf16"

    def __post_init__(self):
        if self.weights not in WEIGHT_FORMATS:
            raise ValueError(f"weights must be one of {WEIGHT_FORMATS}, got {self.weights!r}")
        if self.kv_cache not in KV_FORMATS:
            raise ValueError(f"kv_cache must be one of {KV_FORMATS}, got {self.kv_cache!r}")
        if self.accumulation not in ("fp32", "float32"):
            raise ValueError("the sm_100a kernels accumulate in fp32 only")
        to_torch_dtype(self.activations)
        to_torch_dtype(self.scales)

    @property
    def activation_dtype(self) -> torch.dtype:
        return to_torch_dtype(self.activations)

    @property
    def scale_dtype(self) -> torch.dtype:
        return to_torch_dtype(self.scales)

    @property
    def kv_torch_dtype(self) -> torch.dtype:
        """Storage dtype of KV values (fp4 KV packs two codes per uint8)."""
        return torch.uint8 if self.kv_cache == "fp4" else to_torch_dtype(self.kv_cache)

    def kv_bytes_per_element(self) -> float:
        return {"bf16": 2, "fp16": 2, "fp8": 1, "fp8_e5m2": 1, "int8": 1, "fp4": 0.5}[self.kv_cache]

    def with_(self, **kw) -> "DTypeConfig":
        return replace(self, **kw)


PRESETS: Dict[str, DTypeConfig] = {
    "default": DTypeConfig(),
    "fp16": DTypeConfig(activations="fp16", kv_cache="fp16"),
    "bf16": DTypeConfig(activations="bf16", kv_cache="bf16"),
    "memory_efficient": DTypeConfig(kv_cache="fp8"),
    "long_context": DTypeConfig(kv_cache="fp8"),
    "max_compression": DTypeConfig(kv_cache="fp4"),
    "int8_kv": DTypeConfig(kv_cache="int8"),
}


def get_dtype_config(name: str = "default") -> DTypeConfig:
    try:
        return PRESETS[name]
    except KeyError:
        raise ValueError(f"unknown dtype preset {name!r}; known: {sorted(PRESETS)}") from None
