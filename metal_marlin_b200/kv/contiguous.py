"""Contiguous (non-paged) KV caches: per-layer K/V tensors and the MLA latent cache, with quantized storage
modes, sliding-window eviction, snapshot / restore and automatic growth.

Parity: reference ``metal_marlin/kv_cache.py`` — ``KVCacheTorch`` (``:165``; BHSD / BSHD layouts, fp16 / bf16 /
fp8 / fp8_e5m2 / fp4 / int8 storage, sliding eviction), ``MLAKVCache`` (``:1267``; latent ``[L, B, S, R + dr]``,
quantized modes, ``update_compressed`` ``:1874``, auto-grow ``:2133``, snapshot / restore ``:2175-2200``) and
``metal_marlin/cache/quantized_kv.py`` (FP8 / INT8 compress / decompress).  The paged pool
(``kv/paged.py`` + ``PagedKVStorage``) is what the serving engine uses; these caches back the single-stream
pipelines, the speculative-decoding draft models and ``PersistentKVCache`` prefix reuse.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch

from .._compat import E2M1_VALUES

_FP8_MAX = {"fp8": 448.0, "fp8_e5m2": 57344.0}


# ------------------------------------------------------------------------------------------ quantized storage
def quantize_kv(x: torch.Tensor, mode: str, group: int = 64) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """``x [..., D]`` -> ``(stored, scales)``.  fp8: per-row absmax scale (fp16) + e4m3 / e5m2 bytes; int8:
    per-row symmetric; fp4: E2M1 codes, two per byte, scale per ``group`` features."""
    if mode in ("bf16", "fp16"):
        return x.to(torch.bfloat16 if mode == "bf16" else torch.float16), None
    xf = x.to(torch.float32)
    if mode in _FP8_MAX:
        s = (xf.abs().amax(-1, keepdim=True) / _FP8_MAX[mode]).clamp_min(1e-12)
        dt = torch.float8_e4m3fn if mode == "fp8" else torch.float8_e5m2
        return (xf / s).to(dt), s.to(torch.float16)
    if mode == "int8":
        s = (xf.abs().amax(-1, keepdim=True) / 127.0).clamp_min(1e-12)
        return torch.round(xf / s).clamp(-127, 127).to(torch.int8), s.to(torch.float16)
    if mode == "fp4":
        D = xf.shape[-1]
        g = group if D % group == 0 else D
        xg = xf.reshape(*xf.shape[:-1], D // g, g)
        s = (xg.abs().amax(-1, keepdim=True) / 6.0).clamp_min(1e-12)
        table = torch.tensor(E2M1_VALUES[:8], dtype=torch.float32, device=x.device)
        mag = (xg / s).abs()
        code = (mag.unsqueeze(-1) - table).abs().argmin(-1).to(torch.uint8)
        code = code | ((xg < 0).to(torch.uint8) << 3)
        code = code.reshape(*xf.shape[:-1], D)
        packed = code[..., 0::2] | (code[..., 1::2] << 4)
        return packed, s.squeeze(-1).to(torch.float16)
    raise ValueError(f"unknown KV storage mode {mode!r}")


def dequantize_kv(stored: torch.Tensor, scales: Optional[torch.Tensor], mode: str, dtype=torch.bfloat16) -> torch.Tensor:
    if mode in ("bf16", "fp16"):
        return stored.to(dtype)
    if mode in _FP8_MAX or mode == "int8":
        return (stored.to(torch.float32) * scales.to(torch.float32)).to(dtype)
    if mode == "fp4":
        lo, hi = stored & 0xF, stored >> 4
        code = torch.stack([lo, hi], -1).flatten(-2).long()
        table = torch.tensor(E2M1_VALUES, dtype=torch.float32, device=stored.device)
        v = table[code]
        D = v.shape[-1]
        G = scales.shape[-1]
        v = v.reshape(*v.shape[:-1], G, D // G) * scales.to(torch.float32).unsqueeze(-1)
        return v.reshape(*v.shape[:-2], D).to(dtype)
    raise ValueError(mode)


@dataclass
class CacheConfig:
    num_layers: int
    num_kv_heads: int
    head_dim: int
    max_seq_len: int = 4096
    batch_size: int = 1
    dtype: str = "bf16"                 # bf16 | fp16 | fp8 | fp8_e5m2 | int8 | fp4
    layout: str = "BHSD"                # or BSHD
    sliding_window: int = 0             # > 0: keep only the last `sliding_window` tokens (+ sink tokens)
    sink_tokens: int = 0
    v_head_dim: Optional[int] = None


class KVCache:
    """Per-layer contiguous K/V with ``update(layer, k, v) -> (k_all, v_all)``; positions are tracked per cache
    (all sequences of the batch advance together, as in the single-stream pipelines)."""

    def __init__(self, cfg: CacheConfig, device="cpu"):
        self.cfg = cfg
        self.device = torch.device(device)
        self.seq_len = 0
        self.total_seen = 0
        dv = cfg.v_head_dim or cfg.head_dim
        self._k = [self._alloc(cfg.head_dim) for _ in range(cfg.num_layers)]
        self._v = [self._alloc(dv) for _ in range(cfg.num_layers)]

    # storage: (values, scales)
    def _alloc(self, D: int):
        c = self.cfg
        shape = (c.batch_size, c.num_kv_heads, c.max_seq_len, D) if c.layout == "BHSD" else (c.batch_size, c.max_seq_len, c.num_kv_heads, D)
        vals, sc = quantize_kv(torch.zeros(*shape, device=self.device), c.dtype)
        return [vals, sc]

    def _seq_dim(self) -> int:
        return 2 if self.cfg.layout == "BHSD" else 1

    def _write(self, store, x: torch.Tensor, pos: int):
        vals, sc = quantize_kv(x, self.cfg.dtype)
        T = x.shape[self._seq_dim()]
        sl = [slice(None)] * 4
        sl[self._seq_dim()] = slice(pos, pos + T)
        store[0][tuple(sl)] = vals
        if sc is not None:
            store[1][tuple(sl)] = sc

    def _read(self, store, n: int, dtype) -> torch.Tensor:
        sl = [slice(None)] * 4
        sl[self._seq_dim()] = slice(0, n)
        sc = store[1][tuple(sl)] if store[1] is not None else None
        return dequantize_kv(store[0][tuple(sl)], sc, self.cfg.dtype, dtype)

    def _evict(self, need: int):
        """Sliding eviction: drop the oldest non-sink tokens of every layer so ``need`` more fit."""
        c = self.cfg
        limit = c.sliding_window if c.sliding_window > 0 else c.max_seq_len
        limit = min(limit, c.max_seq_len)
        drop = self.seq_len + need - limit
        if drop <= 0:
            return
        if c.sliding_window <= 0:
            raise RuntimeError(f"KV cache full: {self.seq_len} + {need} > {c.max_seq_len} (no sliding window configured)")
        d = self._seq_dim()
        keep_from = c.sink_tokens + drop
        for store in self._k + self._v:
            for t in store:
                if t is None:
                    continue
                src = t.narrow(d, keep_from, self.seq_len - keep_from).clone()
                t.narrow(d, c.sink_tokens, src.shape[d]).copy_(src)
        self.seq_len -= drop

    def update(self, layer: int, k: torch.Tensor, v: torch.Tensor, dtype=torch.bfloat16):
        """Append ``k, v`` (cache layout, new tokens on the sequence axis) for ``layer``; returns all cached
        K / V of the layer.  The position advances when the last layer is written."""
        T = k.shape[self._seq_dim()]
        if layer == 0:
            self._evict(T)
        self._write(self._k[layer], k, self.seq_len)
        self._write(self._v[layer], v, self.seq_len)
        n = self.seq_len + T
        out = self._read(self._k[layer], n, dtype), self._read(self._v[layer], n, dtype)
        if layer == self.cfg.num_layers - 1:
            self.seq_len = n
            self.total_seen += T
        return out

    def get(self, layer: int, dtype=torch.bfloat16):
        return self._read(self._k[layer], self.seq_len, dtype), self._read(self._v[layer], self.seq_len, dtype)

    def truncate(self, n: int):
        self.seq_len = min(self.seq_len, n)

    def reset(self):
        self.seq_len = 0
        self.total_seen = 0

    def snapshot(self) -> Dict:
        n, d = self.seq_len, self._seq_dim()
        cp = lambda store: [None if t is None else t.narrow(d, 0, n).clone() for t in store]
        return {"seq_len": n, "total_seen": self.total_seen, "k": [cp(s) for s in self._k], "v": [cp(s) for s in self._v]}

    def restore(self, snap: Dict):
        d = self._seq_dim()
        n = snap["seq_len"]
        for dst, src in list(zip(self._k, snap["k"])) + list(zip(self._v, snap["v"])):
            for t, s in zip(dst, src):
                if t is not None:
                    t.narrow(d, 0, n).copy_(s)
        self.seq_len, self.total_seen = n, snap["total_seen"]

    def memory_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for s in self._k + self._v for t in s if t is not None)


KVCacheTorch = KVCache      # reference name


class MLAKVCache:
    """Latent cache ``[L, B, S, R + dr]`` (post-norm c_kv | post-RoPE k_rope rows) with optional quantized
    storage and geometric growth."""

    def __init__(self, num_layers: int, kv_lora_rank: int, rope_dim: int, batch_size: int = 1, max_seq_len: int = 4096,
                 dtype: str = "bf16", device="cpu", initial_seq_len: Optional[int] = None, growth: float = 2.0):
        self.L, self.R, self.dr, self.B = num_layers, kv_lora_rank, rope_dim, batch_size
        self.max_seq_len, self.mode, self.device, self.growth = max_seq_len, dtype, torch.device(device), growth
        self.capacity = min(max_seq_len, initial_seq_len or max_seq_len)
        self.seq_len = 0
        self._vals, self._scales = self._alloc(self.capacity)

    def _alloc(self, cap: int):
        return quantize_kv(torch.zeros(self.L, self.B, cap, self.R + self.dr, device=self.device), self.mode)

    def _grow(self, need: int):
        if need <= self.capacity:
            return
        if need > self.max_seq_len:
            raise RuntimeError(f"MLA cache full: need {need} > max_seq_len {self.max_seq_len}")
        cap = self.capacity
        while cap < need:
            cap = min(self.max_seq_len, max(cap + 1, int(cap * self.growth)))
        vals, sc = self._alloc(cap)
        vals[:, :, : self.seq_len] = self._vals[:, :, : self.seq_len]
        if sc is not None:
            sc[:, :, : self.seq_len] = self._scales[:, :, : self.seq_len]
        self._vals, self._scales, self.capacity = vals, sc, cap

    def update_compressed(self, layer: int, latent: torch.Tensor, dtype=torch.bfloat16) -> torch.Tensor:
        """Append latent rows ``[B, T, R + dr]`` for ``layer`` and return the layer's rows ``[B, S, R + dr]``."""
        T = latent.shape[1]
        self._grow(self.seq_len + T)
        vals, sc = quantize_kv(latent, self.mode)
        self._vals[layer, :, self.seq_len: self.seq_len + T] = vals
        if sc is not None:
            self._scales[layer, :, self.seq_len: self.seq_len + T] = sc
        n = self.seq_len + T
        if layer == self.L - 1:
            self.seq_len = n
        return dequantize_kv(self._vals[layer, :, :n], None if self._scales is None else self._scales[layer, :, :n], self.mode, dtype)

    def get(self, layer: int, dtype=torch.bfloat16) -> torch.Tensor:
        n = self.seq_len
        return dequantize_kv(self._vals[layer, :, :n], None if self._scales is None else self._scales[layer, :, :n], self.mode, dtype)

    def snapshot(self) -> Dict:
        n = self.seq_len
        return {"seq_len": n, "vals": self._vals[:, :, :n].clone(), "scales": None if self._scales is None else self._scales[:, :, :n].clone()}

    def restore(self, snap: Dict):
        n = snap["seq_len"]
        self._grow(n)
        self._vals[:, :, :n] = snap["vals"]
        if self._scales is not None:
            self._scales[:, :, :n] = snap["scales"]
        self.seq_len = n

    def truncate(self, n: int):
        self.seq_len = min(self.seq_len, n)

    def reset(self):
        self.seq_len = 0

    def memory_bytes(self) -> int:
        return self._vals.numel() * self._vals.element_size() + (0 if self._scales is None else self._scales.numel() * 2)


class PersistentKVCache:
    """Prefix-matched cache reuse across calls (reference ``metal_marlin/inference/mmfp4_pipeline.py:31``):
    remembers the token ids whose KV is cached; a new prompt only needs prefill for the tokens after the longest
    common prefix."""

    def __init__(self, cache):
        self.cache = cache
        self.tokens: List[int] = []

    def match(self, prompt: List[int]) -> int:
        """Number of leading prompt tokens already cached (at least one token is always left to prefill)."""
        n = 0
        for a, b in zip(self.tokens, prompt):
            if a != b:
                break
            n += 1
        n = min(n, len(prompt) - 1)
        if n < len(self.tokens):
            self.cache.truncate(n)
            self.tokens = self.tokens[:n]
        return n

    def extend(self, new_tokens: List[int]):
        self.tokens.extend(int(t) for t in new_tokens)

    def reset(self):
        self.tokens = []
        self.cache.reset()
