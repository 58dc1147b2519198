"""Kernel-selection auto-tuner: measures where this engine's dispatch thresholds belong on the GPU it runs on.

Every projection and expert MLP exists as more than one kernel (a weight-streaming kernel for few tokens, an
expert-sorted streaming kernel for a few dozen, the tcgen05 GEMM above that; two attention kernels for prompts), and
``ops`` picks one by token count against module-level thresholds.  The tuner times the candidates on the shapes of a
model, finds the token counts at which the faster kernel changes, and writes a JSON table; ``apply_config`` installs a
table into ``ops`` (global thresholds plus a per-shape limit for dense projections), ``load_config`` reads the table
named by ``$MMB200_TUNING_FILE`` or the per-device file in the cache directory.  ``OnlineAdapter`` keeps running
averages of step times per variant while serving and switches when another variant has become faster.

Parity: reference ``metal_marlin/trellis/autotune_mixed_bpw.py`` (``MixedBPWAutoTuner``: benchmark kernel variants per
batch size / bit width / hidden size, lookup table, per-device cache, online adaptation, JSON export / import,
``get_optimal_config``) and ``metal_marlin/autotuning.py``-style tile sweeps; the tunables here are kernel choices and
token tiles, since a tcgen05 tile is fixed by the instruction shape rather than by a threadgroup size.
"""
from __future__ import annotations

import contextlib
import json
import os
import statistics
from dataclasses import asdict, dataclass, field
from typing import Callable, Dict, Iterable, List, Optional, Sequence, Tuple

import torch

THRESHOLDS = ("GEMV_MAX_M", "MOE_GEMV_MAX_T", "MOE_GROUPED_GEMV_MAX_T", "FMHA_MIN_T")
DEFAULT_BATCHES = (1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128, 192, 256)
_BIG = 1 << 30


@contextlib.contextmanager
def override(**values):
    """Temporarily set dispatch thresholds of ``ops`` (the kernels read them at call time)."""
    from . import ops
    old = {k: getattr(ops, k) for k in values}
    try:
        for k, v in values.items():
            setattr(ops, k, v)
        yield
    finally:
        for k, v in old.items():
            setattr(ops, k, v)


def cuda_timer(iters: int = 20, warmup: int = 3, flush_bytes: int = 256 << 20) -> Callable[[Callable[[], None]], float]:
    """``timer(fn) -> microseconds``: median over ``iters`` runs timed with CUDA events on the current stream, a buffer
    larger than L2 written between runs so that every run starts from device memory."""
    flush = torch.empty(flush_bytes, dtype=torch.uint8, device="cuda")

    def timer(fn: Callable[[], None]) -> float:
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        times = []
        for _ in range(iters):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            b.synchronize()
            times.append(a.elapsed_time(b) * 1e3)
        return statistics.median(times)
    return timer


def crossover(batches: Sequence[int], t_small: Sequence[float], t_large: Sequence[float], tolerance: float = 0.03) -> int:
    """Largest batch up to which the small-batch kernel is at least as fast (within ``tolerance``) at every measured
    batch; 0 if it never is.  A single noisy win beyond the first loss is ignored: thresholds must be monotone."""
    best = 0
    for b, a, c in zip(batches, t_small, t_large):
        if a <= c * (1.0 + tolerance):
            best = b
        else:
            break
    return best


@dataclass
class TunedConfig:
    device: str = "unknown"
    thresholds: Dict[str, int] = field(default_factory=dict)
    linear_limits: Dict[str, int] = field(default_factory=dict)       # "NxK" -> largest token count on the streaming kernel
    moe_token_tiles: Dict[str, int] = field(default_factory=dict)     # "T" -> token tile of the grouped GEMM
    measurements: List[Dict] = field(default_factory=list)

    def save(self, path: str):
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        with open(path, "w") as f:
            json.dump(asdict(self), f, indent=1, sort_keys=True)

    @classmethod
    def load(cls, path: str) -> "TunedConfig":
        with open(path) as f:
            d = json.load(f)
        return cls(**{k: d[k] for k in ("device", "thresholds", "linear_limits", "moe_token_tiles", "measurements") if k in d})


def _random_fp4(out_f: int, in_f: int, gs: int, device, experts: int = 0):
    """Random weights drawn in the quantized domain (no float matrix is ever built)."""
    from .ops.weights import FP4ExpertBank, FP4Weight
    lead = (experts,) if experts else ()
    g = torch.Generator(device="cpu").manual_seed(out_f * 31 + in_f)
    q = torch.randint(-2 ** 31, 2 ** 31 - 1, (*lead, out_f // 16, in_f // 64, 32, 4), dtype=torch.int32, generator=g).to(device)
    s = torch.full((*lead, out_f // 16, in_f // gs, 8, 2), 0.01, dtype=torch.float16, device=device)
    return (FP4ExpertBank if experts else FP4Weight)(q, s, out_f, in_f, gs)


class KernelAutoTuner:
    """Times the kernel variants behind ``ops.linear``, ``ops.moe_forward`` and the prompt attention and derives the
    thresholds.  ``timer`` maps a closure to microseconds (default: CUDA events with an L2 flush); tests pass a model."""

    def __init__(self, device=None, timer: Optional[Callable[[Callable[[], None]], float]] = None,
                 batch_sizes: Sequence[int] = DEFAULT_BATCHES, tolerance: float = 0.03, min_tensor_core_tokens: int = 8):
        self.device = torch.device(device if device is not None else ("cuda" if torch.cuda.is_available() else "cpu"))
        self.timer = timer
        self.batch_sizes = tuple(sorted(batch_sizes))
        self.tolerance = tolerance
        # below this many tokens only the streaming kernels are timed (the tensor-core kernels cannot win there)
        self.min_tc = min_tensor_core_tokens
        name = torch.cuda.get_device_name(self.device) if self.device.type == "cuda" else "cpu"
        self.config = TunedConfig(device=name)

    def _time(self, fn) -> float:
        if self.timer is None:
            self.timer = cuda_timer()
        return float(self.timer(fn))

    def _note(self, **kw):
        self.config.measurements.append(kw)

    # ------------------------------------------------------------------------------------------ dense projections
    def tune_linear(self, shapes: Iterable[Tuple[int, int]], group_size: int = 128) -> Dict[str, int]:
        """For every ``(out, in)``: the largest token count at which the weight-streaming kernel still beats the tcgen05
        GEMM.  The global ``GEMV_MAX_M`` becomes the smallest of them (never slower than tuned on any shape that has no
        entry of its own)."""
        from . import ops
        limits = {}
        for out_f, in_f in shapes:
            W = _random_fp4(out_f, in_f, group_size, self.device)
            t_stream, t_gemm = [], []
            for m in self.batch_sizes:
                x = torch.randn(m, in_f, device=self.device).to(torch.bfloat16)
                with override(GEMV_MAX_M=_BIG, GEMV_LIMITS={}, GEMV_BIG_WEIGHT=_BIG * _BIG):
                    a = self._time(lambda: ops.linear(x, W))
                b = float("inf")
                if m >= self.min_tc:
                    with override(GEMV_MAX_M=0, GEMV_LIMITS={}, GEMV_BIG_WEIGHT=_BIG * _BIG):
                        b = self._time(lambda: ops.linear(x, W))
                t_stream.append(a)
                t_gemm.append(b)
                self._note(kind="linear", shape=f"{out_f}x{in_f}", tokens=m, stream_us=round(a, 2), gemm_us=round(b, 2) if b < 1e30 else None)
            limits[f"{out_f}x{in_f}"] = crossover(self.batch_sizes, t_stream, t_gemm, self.tolerance)
        self.config.linear_limits.update(limits)
        if limits:
            self.config.thresholds["GEMV_MAX_M"] = min(self.config.linear_limits.values())
        return limits

    # ------------------------------------------------------------------------------------------ expert MLPs
    def tune_moe(self, hidden: int, inter: int, num_experts: int, topk: int, group_size: int = 128,
                 token_tiles: Sequence[int] = (32, 64, 128, 256)) -> Tuple[int, int]:
        """The two thresholds of ``ops.moe_forward`` (per-slot streaming -> expert-sorted streaming -> grouped GEMM) and the
        best token tile of the grouped GEMM per token count."""
        from . import ops
        gate_up = _random_fp4(2 * inter, hidden, group_size, self.device, experts=num_experts)
        down = _random_fp4(hidden, inter, group_size, self.device, experts=num_experts)
        t_slot, t_sorted, t_gemm = [], [], []
        g = torch.Generator(device="cpu").manual_seed(7)
        for T in self.batch_sizes:
            x = torch.randn(T, hidden, device=self.device).to(torch.bfloat16)
            ids = torch.stack([torch.randperm(num_experts, generator=g)[:topk] for _ in range(T)]).to(torch.int32).to(self.device)
            w = torch.full((T, topk), 1.0 / topk, dtype=torch.float32, device=self.device)
            with override(MOE_GEMV_MAX_T=_BIG):
                a = self._time(lambda: ops.moe_forward(x, gate_up, down, ids, w))
            b, per_tile = float("inf"), {}
            if T >= 2 * self.min_tc:
                with override(MOE_GEMV_MAX_T=0, MOE_GROUPED_GEMV_MAX_T=_BIG):
                    b = self._time(lambda: ops.moe_forward(x, gate_up, down, ids, w))
                with override(MOE_GEMV_MAX_T=0, MOE_GROUPED_GEMV_MAX_T=0, MOE_TOKEN_TILES=[]):
                    for tt in token_tiles:
                        per_tile[tt] = self._time(lambda tt=tt: ops.moe_forward(x, gate_up, down, ids, w, token_tile=tt))
                best_tile = min(per_tile, key=per_tile.get)
                self.config.moe_token_tiles[str(T)] = best_tile
            t_slot.append(a)
            t_sorted.append(b)
            t_gemm.append(per_tile[best_tile] if per_tile else float("inf"))
            self._note(kind="moe", tokens=T, slot_us=round(a, 2), sorted_us=round(b, 2) if per_tile else None,
                       gemm_us={str(k): round(v, 2) for k, v in per_tile.items()})
        rest = [min(b, c) for b, c in zip(t_sorted, t_gemm)]
        slot_max = crossover(self.batch_sizes, t_slot, rest, self.tolerance)
        sorted_max = max(slot_max, crossover(self.batch_sizes, [min(a, b) for a, b in zip(t_slot, t_sorted)], t_gemm, self.tolerance))
        self.config.thresholds["MOE_GEMV_MAX_T"] = slot_max
        self.config.thresholds["MOE_GROUPED_GEMV_MAX_T"] = sorted_max
        return slot_max, sorted_max

    # ------------------------------------------------------------------------------------------ prompt attention
    def tune_attention(self, heads: int, kv_heads: int, head_dim: int, lengths: Sequence[int] = (128, 256, 384, 512, 1024, 2048)) -> int:
        """Shortest prompt from which the tcgen05 attention kernel beats the mma.sync one (``FMHA_MIN_T``)."""
        from . import ops
        lengths = tuple(sorted(lengths))
        t_sync, t_tc = [], []
        for t in lengths:
            q = torch.randn(t, heads, head_dim, device=self.device).to(torch.bfloat16)
            k = torch.randn(t, kv_heads, head_dim, device=self.device).to(torch.bfloat16)
            v = torch.randn(t, kv_heads, head_dim, device=self.device).to(torch.bfloat16)
            cu = torch.tensor([0, t], dtype=torch.int32, device=self.device)
            with override(FMHA_MIN_T=_BIG):
                a = self._time(lambda: ops.prefill_attention(q, k, v, cu, cu_k=cu, max_q=t))
            with override(FMHA_MIN_T=0):
                b = self._time(lambda: ops.prefill_attention(q, k, v, cu, cu_k=cu, max_q=t))
            t_sync.append(a)
            t_tc.append(b)
            self._note(kind="attention", tokens=t, heads=heads, dim=head_dim, mma_sync_us=round(a, 2), tcgen05_us=round(b, 2))
        keep = crossover(lengths, t_sync, t_tc, self.tolerance)        # longest prompt still better on the mma.sync kernel
        later = [t for t in lengths if t > keep]
        self.config.thresholds["FMHA_MIN_T"] = later[0] if later else _BIG
        return self.config.thresholds["FMHA_MIN_T"]

    # ------------------------------------------------------------------------------------------ whole model
    def run_autotune(self, cfg, attention: bool = True) -> TunedConfig:
        """Tune on the shapes of a model configuration (``models.config.ModelConfig``)."""
        h = cfg.hidden_size
        shapes = set()
        if getattr(cfg, "kv_lora_rank", 0):
            if cfg.q_lora_rank:
                shapes.add(((cfg.q_lora_rank + cfg.kv_lora_rank + cfg.qk_rope_head_dim + 15) // 16 * 16, h))
                shapes.add((cfg.num_attention_heads * (cfg.qk_nope_head_dim + cfg.qk_rope_head_dim), cfg.q_lora_rank))
            shapes.add((h, cfg.num_attention_heads * cfg.v_head_dim))
        else:
            shapes.add(((cfg.num_attention_heads + 2 * cfg.num_key_value_heads) * cfg.dh, h))
            shapes.add((h, cfg.num_attention_heads * cfg.dh))
        if cfg.intermediate_size:
            shapes.add((2 * cfg.intermediate_size, h))
            shapes.add((h, cfg.intermediate_size))
        shapes = sorted(s for s in shapes if s[0] % 16 == 0 and s[1] % 64 == 0)
        gs = getattr(cfg, "group_size", 128) or 128
        self.tune_linear(shapes, gs)
        if getattr(cfg, "num_experts", 0):
            self.tune_moe(h, cfg.moe_intermediate_size, cfg.num_experts, cfg.num_experts_per_tok, gs)
        if attention and not getattr(cfg, "kv_lora_rank", 0) and cfg.dh in (128, 256):
            self.tune_attention(cfg.num_attention_heads, cfg.num_key_value_heads, cfg.dh)
        return self.config

    def export_config(self, path: str):
        self.config.save(path)


# ---------------------------------------------------------------------------------------------- installing a table
def default_path(device_name: Optional[str] = None) -> str:
    if device_name is None:
        device_name = torch.cuda.get_device_name(0) if torch.cuda.is_available() else "cpu"
    base = os.environ.get("MMB200_CACHE_DIR", os.path.join(os.path.expanduser("~"), ".cache", "metal_marlin_b200"))
    return os.path.join(base, "tuning-" + "".join(c if c.isalnum() else "-" for c in device_name) + ".json")


def apply_config(cfg: TunedConfig) -> Dict[str, int]:
    """Install thresholds, per-shape projection limits and grouped-GEMM token tiles into ``ops``; returns what was set."""
    from . import ops
    done = {}
    for k, v in cfg.thresholds.items():
        if k in THRESHOLDS:
            setattr(ops, k, int(v))
            done[k] = int(v)
    ops.GEMV_LIMITS = {tuple(int(a) for a in key.split("x")): int(v) for key, v in cfg.linear_limits.items()}
    ops.MOE_TOKEN_TILES = sorted((int(t), int(tile)) for t, tile in cfg.moe_token_tiles.items())
    return done


def load_config(path: Optional[str] = None, apply: bool = True) -> Optional[TunedConfig]:
    """Read ``path``, else ``$MMB200_TUNING_FILE``, else the per-device file in the cache directory; None if absent."""
    path = path or os.environ.get("MMB200_TUNING_FILE") or default_path()
    if not os.path.isfile(path):
        return None
    cfg = TunedConfig.load(path)
    if apply:
        apply_config(cfg)
    return cfg


def get_optimal_config(tokens: int, out_features: int, in_features: int) -> Dict[str, object]:
    """Which kernel a dense FP4 projection of this shape takes for ``tokens`` rows under the installed table."""
    from . import ops
    lim = ops.GEMV_LIMITS.get((out_features, in_features))
    if lim is None:
        lim = min(ops.GEMV_MAX_M, ops.GEMV_BIG_MAX_M) if out_features * in_features >= ops.GEMV_BIG_WEIGHT else ops.GEMV_MAX_M
    return {"kernel": "fp4_gemv" if tokens <= lim else "fp4_gemm_tcgen05", "limit": lim,
            "tuned": (out_features, in_features) in ops.GEMV_LIMITS}


class OnlineAdapter:
    """Running comparison of interchangeable variants while serving: ``choose(key)`` returns the variant to run (every
    variant a few times first, afterwards the one with the lowest exponential moving average, with a periodic re-probe of
    the others), ``observe(key, variant, us)`` feeds a measured time back."""

    def __init__(self, variants: Sequence[str], alpha: float = 0.2, min_samples: int = 3, reprobe_every: int = 200):
        self.variants = tuple(variants)
        self.alpha, self.min_samples, self.reprobe_every = alpha, min_samples, reprobe_every
        self.ema: Dict[Tuple, float] = {}
        self.count: Dict[Tuple, int] = {}
        self.calls: Dict[object, int] = {}

    def observe(self, key, variant: str, us: float):
        k = (key, variant)
        self.count[k] = self.count.get(k, 0) + 1
        self.ema[k] = us if k not in self.ema else (1 - self.alpha) * self.ema[k] + self.alpha * us

    def choose(self, key) -> str:
        n = self.calls[key] = self.calls.get(key, 0) + 1
        for v in self.variants:
            if self.count.get((key, v), 0) < self.min_samples:
                return v
        best = min(self.variants, key=lambda v: self.ema[(key, v)])
        if self.reprobe_every and n % self.reprobe_every == 0:
            others = [v for v in self.variants if v != best]
            if others:
                return others[(n // self.reprobe_every) % len(others)]
        return best

    def best(self, key) -> Optional[str]:
        seen = [v for v in self.variants if (key, v) in self.ema]
        return min(seen, key=lambda v: self.ema[(key, v)]) if seen else None
