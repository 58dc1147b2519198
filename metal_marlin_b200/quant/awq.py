"""AWQ: activation-aware per-input-channel scaling searched on a grid before group quantization.

Parity: reference ``metal_marlin/awq.py`` (per-channel scale ``s = mean|x|^alpha``, ``alpha`` searched over a
grid to minimise the output error on calibration activations; the scale is folded into the weight and its
inverse into the producer of the activation).
"""
from __future__ import annotations

from typing import Callable, Dict, Tuple

import torch

from .rtn import quantize as rtn_quantize


def awq_search(w: torch.Tensor, x: torch.Tensor, fmt: str = "fp4", group_size: int = 128, n_grid: int = 20) -> Tuple[torch.Tensor, Dict]:
    """``w [out, in]``, calibration activations ``x [n, in]``.  Returns the per-channel scale ``s [in]`` (the layer
    becomes ``(W * s) (x / s)``) and search statistics."""
    W = w.to(torch.float32)
    X = x.to(torch.float32)
    ref = X @ W.t()
    act = X.abs().mean(0).clamp_min(1e-8)
    best, best_err, best_alpha = torch.ones_like(act), float("inf"), 0.0
    for i in range(n_grid + 1):
        alpha = i / n_grid
        s = act.pow(alpha)
        s = s / (s.max() * s.min()).sqrt()
        wq = rtn_quantize(W * s, fmt, group_size).dequantize(torch.float32) / s
        err = float(((X @ wq.t()) - ref).pow(2).mean())
        if err < best_err:
            best, best_err, best_alpha = s, err, alpha
    base = float(((X @ rtn_quantize(W, fmt, group_size).dequantize(torch.float32).t()) - ref).pow(2).mean())
    return best, {"alpha": best_alpha, "mse": best_err, "mse_rtn": base}


def awq_quantize(w: torch.Tensor, x: torch.Tensor, fmt: str = "fp4", group_size: int = 128, n_grid: int = 20):
    """Returns ``(QuantizedTensor of W * s, s, stats)``."""
    s, stats = awq_search(w, x, fmt, group_size, n_grid)
    return rtn_quantize(w.to(torch.float32) * s, fmt, group_size), s, stats
