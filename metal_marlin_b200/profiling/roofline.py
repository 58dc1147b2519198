"""Roofline arithmetic against the measured peaks of the machine, FLOP / byte calculators for the model's ops, and a
CUDA-event kernel timer.

Parity: reference ``metal_marlin/profiling/roofline.py:223`` (ridge point, bound classification, achieved fractions),
``metal_marlin/profile/calculator.py:225`` / ``utils/profile_ops.py`` (FLOP counts of GEMM / attention / MoE layers),
``metal_marlin/profiling/kernel_timer.py`` and the ``@profile_kernel`` decorator (``utils/profiling.py:218``).  The
denominators are the copy bandwidth and bf16 GEMM throughput measured on the target GPUs (``MEASURED_PEAKS.json`` at
the repository root when present, otherwise the documented fallback), not datasheet numbers.
"""
from __future__ import annotations

import functools
import json
import os
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional

import torch

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}
NVLINK_GBS_PER_DIRECTION = 770.0       # measured peer copy; nominal 900


def load_peaks(path: Optional[str] = None) -> Dict[str, float]:
    here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    p = path or os.path.join(here, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d.get("hbm_gbs", FALLBACK_PEAKS["hbm_gbs"])), "bf16_tflops": float(d.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"])),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", FALLBACK_PEAKS["bf16_tflops_sustained"])), "source": "measured"}
    return dict(FALLBACK_PEAKS)


@dataclass
class RooflinePoint:
    name: str
    flops: float
    bytes: float
    seconds: float
    peaks: Dict[str, float]

    @property
    def intensity(self) -> float:
        return self.flops / max(self.bytes, 1.0)

    @property
    def ridge(self) -> float:
        return self.peaks["bf16_tflops"] * 1e12 / (self.peaks["hbm_gbs"] * 1e9)

    @property
    def bound(self) -> str:
        return "compute" if self.intensity >= self.ridge else "memory"

    @property
    def achieved_gbs(self) -> float:
        return self.bytes / self.seconds / 1e9

    @property
    def achieved_tflops(self) -> float:
        return self.flops / self.seconds / 1e12

    @property
    def fraction_of_roof(self) -> float:
        """Achieved / attainable at this arithmetic intensity ("of measured" or "of fallback", see ``peaks['source']``)."""
        roof_time = max(self.flops / (self.peaks["bf16_tflops"] * 1e12), self.bytes / (self.peaks["hbm_gbs"] * 1e9))
        return roof_time / self.seconds

    def row(self) -> Dict:
        return {"name": self.name, "us": self.seconds * 1e6, "GB/s": self.achieved_gbs, "TFLOP/s": self.achieved_tflops, "intensity": self.intensity,
                "bound": self.bound, "fraction": self.fraction_of_roof, "of": self.peaks["source"]}


def fused_collective_roof_seconds(flops: float, nvlink_bytes: float, peaks: Optional[Dict[str, float]] = None) -> float:
    """Target time of a fused compute + collective kernel: the slower of the math and the bytes that must cross NVLink."""
    peaks = peaks or load_peaks()
    return max(flops / (peaks["bf16_tflops"] * 1e12), nvlink_bytes / (NVLINK_GBS_PER_DIRECTION * 1e9))


# ------------------------------------------------------------------------------------------ FLOP / byte calculators
def gemm_flops(m: int, n: int, k: int) -> float:
    return 2.0 * m * n * k


def fp4_weight_bytes(n: int, k: int, group_size: int = 128) -> float:
    return n * k / 2 + n * (k / group_size) * 2


def attention_flops(batch: int, heads: int, q_len: int, kv_len: int, d_qk: int, d_v: int, causal: bool = False) -> float:
    f = 2.0 * batch * heads * q_len * kv_len * (d_qk + d_v)
    return f / 2 if causal and q_len == kv_len else f


def decode_step_cost(cfg, batch: int, ctx: int) -> Dict[str, float]:
    """Algorithmic FLOPs and HBM bytes of one decode step of ``cfg`` (weights streamed once, KV read once)."""
    active = cfg.param_count()["active"] - cfg.vocab_size * cfg.hidden_size      # quantized matrices touched per token
    w_bytes = active * 0.5 * (1 + 4.0 / cfg.group_size) + cfg.vocab_size * cfg.hidden_size * 2
    if cfg.is_mla:
        kv_row = (cfg.kv_lora_rank + cfg.qk_rope_head_dim) * 2
        att = attention_flops(batch, cfg.num_attention_heads, 1, ctx, cfg.kv_lora_rank + cfg.qk_rope_head_dim, cfg.kv_lora_rank)
    else:
        hd = cfg.head_dim or cfg.hidden_size // cfg.num_attention_heads
        kv_row = 2 * cfg.num_key_value_heads * hd * 2
        att = attention_flops(batch, cfg.num_attention_heads, 1, ctx, hd, hd)
    kv_bytes = batch * ctx * kv_row * cfg.num_hidden_layers
    return {"flops": 2.0 * active * batch + att * cfg.num_hidden_layers, "weight_bytes": w_bytes, "kv_bytes": kv_bytes, "bytes": w_bytes + kv_bytes}


# ------------------------------------------------------------------------------------------ timers
class KernelTimer:
    """CUDA-event timing with warm-up; host timing on CPU.  ``time(fn)`` returns the median seconds."""

    def __init__(self, warmup: int = 3, iters: int = 10, flush_l2: bool = True):
        self.warmup, self.iters, self.flush_l2 = warmup, iters, flush_l2
        self._flush = None
        self.records: Dict[str, List[float]] = {}

    def time(self, fn: Callable[[], object], name: str = "") -> float:
        import time as _t
        cuda = torch.cuda.is_available()
        for _ in range(self.warmup):
            fn()
        ts = []
        if cuda:
            if self.flush_l2 and self._flush is None:
                self._flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
            torch.cuda.synchronize()
            for _ in range(self.iters):
                if self.flush_l2:
                    self._flush.fill_(1)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                fn()
                e1.record()
                torch.cuda.synchronize()
                ts.append(e0.elapsed_time(e1) * 1e-3)
        else:
            for _ in range(self.iters):
                t = _t.perf_counter()
                fn()
                ts.append(_t.perf_counter() - t)
        ts.sort()
        med = ts[len(ts) // 2]
        if name:
            self.records.setdefault(name, []).append(med)
        return med


_global_timer = KernelTimer(warmup=0, iters=1, flush_l2=False)
PROFILE_ON = os.environ.get("MM_PROFILE", "0") == "1"


def profile_kernel(name: Optional[str] = None):
    """Decorator: when ``MM_PROFILE=1`` every call is timed (device-synchronised) into ``profile_records()``."""
    def deco(fn):
        label = name or fn.__name__

        @functools.wraps(fn)
        def wrapped(*a, **kw):
            if not PROFILE_ON:
                return fn(*a, **kw)
            out = []
            _global_timer.time(lambda: out.append(fn(*a, **kw)), label)
            return out[-1]
        return wrapped
    return deco


def profile_records() -> Dict[str, List[float]]:
    return _global_timer.records


def get_timer() -> KernelTimer:
    """The process-wide timer behind ``profile_kernel`` (reference ``profiling/kernel_timer.py:62``)."""
    return _global_timer
