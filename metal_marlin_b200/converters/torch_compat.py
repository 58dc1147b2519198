"""4-bit weights between the two packings other PyTorch tooling uses: "Marlin" words hold eight codes along the OUTPUT
dimension (``uint32 [K, N / 8]``), GPTQ / AutoGPTQ words hold eight codes along the INPUT dimension (``int32 [K / 8, N]``); scales
(``[groups, N]``) are shared.  Code ``i`` of a word sits in bits ``4 i .. 4 i + 3`` in both.

Parity: reference ``torch_compat.py`` (``export_for_pytorch`` :22, ``import_from_pytorch`` :70).
"""
from __future__ import annotations

from typing import Any, Dict, Tuple

import numpy as np

_SHIFTS = (np.arange(8, dtype=np.uint32) * 4)


def unpack_along_n(packed: np.ndarray, N: int) -> np.ndarray:
    """``uint32 [K, N / 8] -> uint8 codes [K, N]``."""
    w = np.ascontiguousarray(packed).view(np.uint32)
    return ((w[:, :, None] >> _SHIFTS[None, None, :]) & 0xF).reshape(w.shape[0], -1)[:, :N].astype(np.uint8)


def pack_along_n(codes: np.ndarray) -> np.ndarray:
    K, N = codes.shape
    if N % 8:
        raise ValueError(f"N = {N} is not a multiple of 8")
    c = codes.astype(np.uint32).reshape(K, N // 8, 8)
    return np.bitwise_or.reduce(c << _SHIFTS[None, None, :], axis=2).astype(np.uint32)


def unpack_along_k(qweight: np.ndarray) -> np.ndarray:
    """``int32 [K / 8, N] -> uint8 codes [K, N]``."""
    w = np.ascontiguousarray(qweight).view(np.uint32)
    return ((w[:, None, :] >> _SHIFTS[None, :, None]) & 0xF).reshape(-1, w.shape[1]).astype(np.uint8)


def pack_along_k(codes: np.ndarray) -> np.ndarray:
    K, N = codes.shape
    if K % 8:
        raise ValueError(f"K = {K} is not a multiple of 8")
    c = codes.astype(np.uint32).reshape(K // 8, 8, N)
    return np.bitwise_or.reduce(c << _SHIFTS[None, :, None], axis=1).astype(np.uint32).view(np.int32)


def export_for_pytorch(packed_weights: np.ndarray, scales: np.ndarray, metadata: Dict[str, Any]) -> Dict[str, np.ndarray]:
    """Marlin-packed ``[K, N / 8]`` + scales -> a GPTQ-style state dict (``qweight [K / 8, N]``, ``scales``, ``g_idx [K]``, ``bits``,
    ``group_size``).  ``metadata``: ``in_features`` (K), ``out_features`` (N), ``group_size``."""
    K, N, gs = int(metadata["in_features"]), int(metadata["out_features"]), int(metadata["group_size"])
    if packed_weights.shape != (K, (N + 7) // 8):
        raise ValueError(f"packed weights {packed_weights.shape} do not match K = {K}, N = {N}")
    return {"qweight": pack_along_k(unpack_along_n(packed_weights, N)), "scales": np.asarray(scales).astype(np.float16),
            "g_idx": (np.arange(K, dtype=np.int32) // gs), "bits": np.array([4], dtype=np.int32), "group_size": np.array([gs], dtype=np.int32)}


def import_from_pytorch(state_dict: Dict[str, np.ndarray]) -> Tuple[np.ndarray, np.ndarray, int]:
    """The inverse: ``(packed [K, N / 8], scales [groups, N] fp16, group_size)``; the group size comes from ``group_size`` when present,
    else from the shapes (K over the number of scale rows)."""
    q = np.asarray(state_dict["qweight"])
    scales = np.asarray(state_dict["scales"])
    codes = unpack_along_k(q)
    if "group_size" in state_dict:
        gs = int(np.asarray(state_dict["group_size"]).reshape(-1)[0])
    else:
        gs = codes.shape[0] // max(1, scales.shape[0])
    return pack_along_n(codes), scales.astype(np.float16), gs
