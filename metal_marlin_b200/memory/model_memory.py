"""Model-level memory planning and memory-mapped weights: per-layer and per-expert byte counts of a configuration, the
MLA cache compression ratio, a planner that decides how many experts stay resident under a byte limit, a compaction
wrapper over the arena, and a manager for memory-mapped checkpoint files.

Parity: reference ``metal_marlin/memory/mmfp4_memory.py`` (``MMFP4MemoryManager``, ``LayerMetadata``, ``ExpertMetadata``,
``MLACompressionRatio``, ``MemoryStats``), ``memory/device_memory.py`` (``MemoryCompactor``, ``CompactionConfig``, ``CompactionStats``),
``mmap_loader.py`` (``MMAPWeightManager``, ``MMAPWeightConfig``, ``MMAPWeightStats``), ``memory/cuda_pinned_pool.py`` and
``memory/buffer_pool.py`` (``PooledBuffer``).
"""
from __future__ import annotations

import os
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch

from .arena import Arena
from .streaming import PinnedPool

CUDAPinnedPool = PinnedPool


@dataclass
class PooledBuffer:
    tensor: torch.Tensor
    last_used: float = field(default_factory=time.monotonic)
    use_count: int = 0

    def touch(self) -> None:
        self.last_used = time.monotonic()
        self.use_count += 1


@dataclass
class ExpertMetadata:
    layer: int
    expert: int
    nbytes: int
    resident: bool = True


@dataclass
class LayerMetadata:
    layer: int
    attention_bytes: int
    mlp_bytes: int
    expert_bytes: int = 0            # one routed expert
    num_experts: int = 0

    @property
    def total_bytes(self) -> int:
        return self.attention_bytes + self.mlp_bytes + self.expert_bytes * self.num_experts


@dataclass
class MLACompressionRatio:
    latent_bytes_per_token: float
    full_bytes_per_token: float

    @property
    def ratio(self) -> float:
        return self.full_bytes_per_token / max(self.latent_bytes_per_token, 1e-9)

    @classmethod
    def of(cls, cfg, dtype_bytes: float = 2.0) -> "MLACompressionRatio":
        latent = (cfg.kv_lora_rank + cfg.qk_rope_head_dim) * dtype_bytes
        full = cfg.num_attention_heads * (cfg.qk_nope_head_dim + cfg.qk_rope_head_dim + cfg.v_head_dim) * dtype_bytes
        return cls(latent, full)


@dataclass
class MemoryStats:
    weight_bytes: int
    resident_expert_bytes: int
    offloaded_expert_bytes: int
    kv_bytes_per_token: float
    limit_bytes: int

    @property
    def kv_tokens_that_fit(self) -> int:
        free = self.limit_bytes - self.weight_bytes - self.resident_expert_bytes
        return max(0, int(free // max(self.kv_bytes_per_token, 1e-9)))


class MMFP4MemoryManager:
    """Byte accounting of an FP4 model from its configuration (4-bit codes + one fp16 scale per group), and a residency plan:
    under ``limit_bytes`` dense weights always stay, routed experts stay from the first layer on until the limit is reached
    (the rest would be streamed through ``memory.ExpertCache``)."""

    def __init__(self, cfg, limit_bytes: Optional[int] = None, group_size: Optional[int] = None, kv_dtype_bytes: float = 2.0):
        self.cfg = cfg
        self.gs = group_size or getattr(cfg, "group_size", 128) or 128
        self.limit = limit_bytes if limit_bytes is not None else (torch.cuda.mem_get_info()[1] if torch.cuda.is_available() else 180 << 30)
        self.kv_dtype_bytes = kv_dtype_bytes
        self.layers: List[LayerMetadata] = [self._layer(i) for i in range(cfg.num_hidden_layers)]

    def _w(self, n_params: int) -> int:
        return int(n_params * (0.5 + 2.0 / self.gs))

    def _layer(self, i: int) -> LayerMetadata:
        c, h = self.cfg, self.cfg.hidden_size
        if c.is_mla:
            dq = c.qk_nope_head_dim + c.qk_rope_head_dim
            attn = ((h * c.q_lora_rank + c.q_lora_rank * c.num_attention_heads * dq) if c.q_lora_rank else h * c.num_attention_heads * dq)
            attn += h * (c.kv_lora_rank + c.qk_rope_head_dim) + c.kv_lora_rank * c.num_attention_heads * (c.qk_nope_head_dim + c.v_head_dim)
            attn += c.num_attention_heads * c.v_head_dim * h
        else:
            attn = h * (c.num_attention_heads + 2 * c.num_key_value_heads) * c.dh + c.num_attention_heads * c.dh * h
        if c.layer_is_moe(i):
            e = 3 * h * c.moe_intermediate_size
            return LayerMetadata(i, self._w(attn), self._w(e * c.n_shared_experts) + 2 * h * c.num_experts, self._w(e), c.num_experts)
        return LayerMetadata(i, self._w(attn), self._w(3 * h * c.intermediate_size))

    def kv_bytes_per_token(self) -> float:
        c = self.cfg
        per_layer = ((c.kv_lora_rank + c.qk_rope_head_dim) if c.is_mla else 2 * c.num_key_value_heads * c.dh) * self.kv_dtype_bytes
        return per_layer * c.num_hidden_layers

    def plan(self) -> Dict:
        c = self.cfg
        emb = c.vocab_size * c.hidden_size * 2 * (1 if c.tie_word_embeddings else 2)
        dense = emb + sum(l.attention_bytes + l.mlp_bytes for l in self.layers)
        experts: List[ExpertMetadata] = []
        used = dense
        for l in self.layers:
            for e in range(l.num_experts):
                fits = used + l.expert_bytes <= self.limit
                experts.append(ExpertMetadata(l.layer, e, l.expert_bytes, fits))
                if fits:
                    used += l.expert_bytes
        res = sum(e.nbytes for e in experts if e.resident)
        off = sum(e.nbytes for e in experts if not e.resident)
        return {"stats": MemoryStats(dense, res, off, self.kv_bytes_per_token(), self.limit), "experts": experts,
                "fits_entirely": off == 0 and dense + res <= self.limit}


@dataclass
class CompactionConfig:
    fragmentation_threshold: float = 0.3      # compact when the largest free block is this much smaller than the free total
    min_interval_s: float = 1.0


@dataclass
class CompactionStats:
    runs: int = 0
    blocks_moved: int = 0
    last_run: float = 0.0


class MemoryCompactor:
    """Compacts an :class:`Arena` when its free space is fragmented; the owner passes ``on_moved(old_offset, new_offset)``
    to refresh its views."""

    def __init__(self, arena: Arena, config: Optional[CompactionConfig] = None, on_moved=None):
        self.arena, self.cfg, self.on_moved, self.stats = arena, config or CompactionConfig(), on_moved, CompactionStats()

    def fragmentation(self) -> float:
        s = self.arena.stats()
        free = s["capacity"] - s["used"]
        return 0.0 if free <= 0 else 1.0 - s["largest_free"] / free

    def maybe_compact(self, force: bool = False) -> int:
        now = time.monotonic()
        if not force and (self.fragmentation() < self.cfg.fragmentation_threshold or now - self.stats.last_run < self.cfg.min_interval_s):
            return 0
        remap = self.arena.compact()
        for old, new in remap.items():
            if old != new and self.on_moved is not None:
                self.on_moved(old, new)
        moved = sum(1 for o, n in remap.items() if o != n)
        self.stats.runs += 1
        self.stats.blocks_moved += moved
        self.stats.last_run = now
        return moved


@dataclass
class MMAPWeightConfig:
    max_open_files: int = 8
    pin: bool = False                 # copy loaded tensors into pinned memory (faster host -> device copies)


@dataclass
class MMAPWeightStats:
    loads: int = 0
    bytes_loaded: int = 0
    files_opened: int = 0


class MMAPWeightManager:
    """Tensors of a checkpoint directory served from memory-mapped safetensors files: nothing is read until a tensor is
    asked for, and the operating system's page cache does the caching."""

    def __init__(self, path: str, config: Optional[MMAPWeightConfig] = None):
        from ..formats.mmfp4_loader import MMFP4ModelLoader
        self.cfg = config or MMAPWeightConfig()
        self._ld = MMFP4ModelLoader(path, prefetch_workers=0, cache_files=self.cfg.max_open_files)
        self.stats = MMAPWeightStats()

    def names(self) -> List[str]:
        return self._ld.tensor_names()

    def get(self, name: str, device=None) -> torch.Tensor:
        t = self._ld.load_tensor(name)
        self.stats.loads += 1
        self.stats.bytes_loaded += t.numel() * t.element_size()
        self.stats.files_opened = len(self._ld._files)
        if self.cfg.pin and torch.cuda.is_available():
            t = t.pin_memory()
        return t if device is None else t.to(device, non_blocking=True)

    def layer(self, index: int, device=None) -> Dict[str, torch.Tensor]:
        return {k: self.get(k, device) for k in self._ld.layer_tensor_names(index)}

    def close(self) -> None:
        self._ld.close()
