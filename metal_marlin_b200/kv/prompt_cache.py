"""Prompt (prefix) caches that keep the KV *contents* of token blocks across requests and across storage tiers.

``TieredPrefixCache`` chains block hashes (block i's hash covers tokens ``0 .. (i + 1) * block_size``), so a lookup walks the
prompt block by block until the first miss.  ``RadixPrefixCache`` keeps the same blocks in a trie keyed by the token
tuple of each block: lookups need no hashing of the whole prefix and a partial last block still reports how many of
its leading tokens match.  Blocks live on the GPU (device tensors), in pinned host RAM, or on disk; GPU overflow is
demoted to RAM, RAM overflow to disk (or dropped), and a hit on a lower tier promotes the block back.

On a B200 box the RAM tier is pinned memory and promotion is one asynchronous H2D copy per block on the caller's stream;
180 GB of HBM make the GPU tier large, the lower tiers matter for multi-tenant prompt libraries.

Parity: reference ``metal_marlin/cache/prompt_cache.py:67-819`` (``StorageTier``, ``PrefixCacheConfig``, ``PrefixMatch``,
``CachedBlock``, ``CacheMetrics``, ``PrefixCache.match_prefix / get_blocks / store_prefix / release_blocks / memory_usage``,
``RadixPrefixCache``).
"""
from __future__ import annotations

import enum
import hashlib
import os
import time
from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch


class StorageTier(enum.Enum):
    GPU = "gpu"
    RAM = "ram"
    DISK = "disk"


@dataclass
class PrefixCacheConfig:
    block_size: int = 16
    max_gpu_blocks: int = 1024
    max_ram_blocks: int = 4096
    disk_path: Optional[str] = None          # None: RAM overflow is dropped
    max_disk_blocks: int = 1 << 16
    device: str = "cpu"                      # device of the GPU tier ("cuda" on a GPU box)
    pin_memory: bool = False                 # pinned RAM tier (needs CUDA)


@dataclass
class PrefixMatch:
    num_tokens: int = 0                      # matched tokens (a multiple of block_size for the hash cache)
    block_hashes: List[str] = field(default_factory=list)
    tiers: List[StorageTier] = field(default_factory=list)
    partial_tokens: int = 0                  # radix cache: leading tokens of the next block that also match

    @property
    def num_blocks(self) -> int:
        return len(self.block_hashes)


@dataclass
class CachedBlock:
    block_hash: str
    tokens: Tuple[int, ...]
    tier: StorageTier
    data: Optional[torch.Tensor]             # the block's KV rows, any shape; None while on disk
    ref_count: int = 0
    last_access: float = field(default_factory=time.monotonic)
    hits: int = 0
    path: Optional[str] = None

    def touch(self) -> None:
        self.last_access = time.monotonic()
        self.hits += 1

    def nbytes(self) -> int:
        return 0 if self.data is None else self.data.numel() * self.data.element_size()


@dataclass
class CacheMetrics:
    lookups: int = 0
    hit_blocks: int = 0
    miss_blocks: int = 0
    promotions: int = 0
    demotions: int = 0
    disk_writes: int = 0
    disk_reads: int = 0
    dropped: int = 0

    def hit_rate(self) -> float:
        tot = self.hit_blocks + self.miss_blocks
        return self.hit_blocks / tot if tot else 0.0

    def reset(self) -> None:
        for k in vars(self):
            setattr(self, k, 0)


def _block_hash(prev: str, tokens: Sequence[int]) -> str:
    h = hashlib.blake2b(digest_size=16)
    h.update(prev.encode())
    h.update(b",".join(str(int(t)).encode() for t in tokens))
    return h.hexdigest()


class TieredPrefixCache:
    """Hash-chained prefix cache over three storage tiers."""

    def __init__(self, config: Optional[PrefixCacheConfig] = None):
        self.cfg = config or PrefixCacheConfig()
        self.blocks: Dict[str, CachedBlock] = {}
        self._gpu: "OrderedDict[str, None]" = OrderedDict()      # LRU order per tier
        self._ram: "OrderedDict[str, None]" = OrderedDict()
        self._disk: "OrderedDict[str, None]" = OrderedDict()
        self.metrics = CacheMetrics()
        if self.cfg.disk_path:
            os.makedirs(self.cfg.disk_path, exist_ok=True)

    # ------------------------------------------------------------------ lookup
    def _chain(self, tokens: Sequence[int]) -> List[Tuple[str, Tuple[int, ...]]]:
        bs, out, prev = self.cfg.block_size, [], ""
        for i in range(0, len(tokens) - len(tokens) % bs, bs):
            blk = tuple(int(t) for t in tokens[i:i + bs])
            prev = _block_hash(prev, blk)
            out.append((prev, blk))
        return out

    def match_prefix(self, tokens: Sequence[int]) -> PrefixMatch:
        self.metrics.lookups += 1
        m = PrefixMatch()
        chain = self._chain(tokens)
        for h, _ in chain:
            b = self.blocks.get(h)
            if b is None:
                break
            m.block_hashes.append(h)
            m.tiers.append(b.tier)
        m.num_tokens = len(m.block_hashes) * self.cfg.block_size
        self.metrics.hit_blocks += len(m.block_hashes)
        self.metrics.miss_blocks += len(chain) - len(m.block_hashes)
        return m

    def get_blocks(self, block_hashes: Sequence[str], acquire: bool = True) -> List[torch.Tensor]:
        """KV tensors of the blocks on the GPU tier's device (lower tiers are promoted); ``acquire`` pins them against
        eviction until :meth:`release_blocks`."""
        out = []
        for h in block_hashes:
            b = self.blocks[h]
            if b.tier is not StorageTier.GPU:
                self._promote_to_gpu(b)
            else:
                self._gpu.move_to_end(h)
            b.touch()
            if acquire:
                b.ref_count += 1
            out.append(b.data)
        return out

    def release_blocks(self, block_hashes: Sequence[str]) -> None:
        for h in block_hashes:
            b = self.blocks.get(h)
            if b is not None and b.ref_count > 0:
                b.ref_count -= 1

    # ------------------------------------------------------------------ insertion
    def store_prefix(self, tokens: Sequence[int], kv_blocks: Sequence[torch.Tensor]) -> int:
        """Cache the full blocks of ``tokens``; ``kv_blocks[i]`` holds the KV rows of block i (copied).  Returns the
        number of newly stored blocks."""
        new = 0
        for (h, blk), data in zip(self._chain(tokens), kv_blocks):
            if h in self.blocks:
                self.blocks[h].touch()
                continue
            b = CachedBlock(h, blk, StorageTier.GPU, data.detach().to(self.cfg.device, copy=True))
            self.blocks[h] = b
            self._add_to_gpu(b)
            new += 1
        return new

    def extend_from_cache(self, tokens: Sequence[int]) -> Tuple[int, List[torch.Tensor]]:
        """(matched tokens, their KV blocks on the device): what a request can skip in its prompt pass."""
        m = self.match_prefix(tokens)
        return m.num_tokens, self.get_blocks(m.block_hashes, acquire=False)

    # ------------------------------------------------------------------ tiers
    def _add_to_gpu(self, b: CachedBlock) -> None:
        b.tier = StorageTier.GPU
        self._gpu[b.block_hash] = None
        while len(self._gpu) > self.cfg.max_gpu_blocks and self._evict_from_gpu():
            pass

    def _victim(self, order: "OrderedDict[str, None]") -> Optional[CachedBlock]:
        for h in order:
            if self.blocks[h].ref_count == 0:
                return self.blocks[h]
        return None

    def _evict_from_gpu(self) -> bool:
        b = self._victim(self._gpu)
        if b is None:
            return False
        del self._gpu[b.block_hash]
        host = b.data.to("cpu")
        if self.cfg.pin_memory and torch.cuda.is_available():
            host = host.pin_memory()
        b.data, b.tier = host, StorageTier.RAM
        self._ram[b.block_hash] = None
        self.metrics.demotions += 1
        while len(self._ram) > self.cfg.max_ram_blocks and self._evict_from_ram():
            pass
        return True

    def _evict_from_ram(self) -> bool:
        b = self._victim(self._ram)
        if b is None:
            return False
        del self._ram[b.block_hash]
        if self.cfg.disk_path:
            self._save_to_disk(b)
            while len(self._disk) > self.cfg.max_disk_blocks:
                h, _ = self._disk.popitem(last=False)
                self._drop(self.blocks[h])
        else:
            self._drop(b)
        return True

    def _drop(self, b: CachedBlock) -> None:
        if b.path and os.path.exists(b.path):
            os.remove(b.path)
        self.blocks.pop(b.block_hash, None)
        self.metrics.dropped += 1

    def _save_to_disk(self, b: CachedBlock) -> None:
        b.path = os.path.join(self.cfg.disk_path, b.block_hash + ".pt")
        torch.save(b.data, b.path)
        b.data, b.tier = None, StorageTier.DISK
        self._disk[b.block_hash] = None
        self.metrics.disk_writes += 1

    def _promote_to_gpu(self, b: CachedBlock) -> None:
        if b.tier is StorageTier.DISK:
            b.data = torch.load(b.path, map_location="cpu")
            self._disk.pop(b.block_hash, None)
            self.metrics.disk_reads += 1
        else:
            self._ram.pop(b.block_hash, None)
        b.data = b.data.to(self.cfg.device, non_blocking=True)
        b.ref_count += 1                      # not a victim of the evictions its own promotion may trigger
        self._add_to_gpu(b)
        b.ref_count -= 1
        self.metrics.promotions += 1

    # ------------------------------------------------------------------ bookkeeping
    def clear(self) -> None:
        for b in list(self.blocks.values()):
            if b.path and os.path.exists(b.path):
                os.remove(b.path)
        self.blocks.clear()
        self._gpu.clear()
        self._ram.clear()
        self._disk.clear()

    def memory_usage(self) -> Dict[str, int]:
        use = {"gpu_blocks": len(self._gpu), "ram_blocks": len(self._ram), "disk_blocks": len(self._disk), "gpu_bytes": 0, "ram_bytes": 0}
        for b in self.blocks.values():
            if b.tier is StorageTier.GPU:
                use["gpu_bytes"] += b.nbytes()
            elif b.tier is StorageTier.RAM:
                use["ram_bytes"] += b.nbytes()
        return use

    def __len__(self) -> int:
        return len(self.blocks)

    def __repr__(self) -> str:
        u = self.memory_usage()
        return f"{type(self).__name__}(gpu={u['gpu_blocks']}, ram={u['ram_blocks']}, disk={u['disk_blocks']}, hit_rate={self.metrics.hit_rate():.2f})"


class _RadixNode:
    __slots__ = ("children", "block_hash")

    def __init__(self):
        self.children: Dict[Tuple[int, ...], "_RadixNode"] = {}
        self.block_hash: Optional[str] = None


class RadixPrefixCache(TieredPrefixCache):
    """Same storage, lookups through a trie whose edges are whole token blocks; reports partial matches of the next block."""

    def __init__(self, config: Optional[PrefixCacheConfig] = None):
        super().__init__(config)
        self.root = _RadixNode()

    def match_prefix(self, tokens: Sequence[int]) -> PrefixMatch:
        self.metrics.lookups += 1
        bs, node, m = self.cfg.block_size, self.root, PrefixMatch()
        n_full = len(tokens) // bs
        i = 0
        while i < n_full:
            key = tuple(int(t) for t in tokens[i * bs:(i + 1) * bs])
            nxt = node.children.get(key)
            if nxt is None or nxt.block_hash not in self.blocks:
                break
            m.block_hashes.append(nxt.block_hash)
            m.tiers.append(self.blocks[nxt.block_hash].tier)
            node = nxt
            i += 1
        m.num_tokens = i * bs
        rest = [int(t) for t in tokens[i * bs:(i + 1) * bs]]
        for key, child in node.children.items():       # longest common lead of the next block (informational)
            if child.block_hash in self.blocks:
                k = 0
                while k < len(rest) and k < len(key) and key[k] == rest[k]:
                    k += 1
                m.partial_tokens = max(m.partial_tokens, k)
        self.metrics.hit_blocks += i
        self.metrics.miss_blocks += n_full - i
        return m

    def store_prefix(self, tokens: Sequence[int], kv_blocks: Sequence[torch.Tensor]) -> int:
        new = super().store_prefix(tokens, kv_blocks)
        node = self.root
        for (h, blk), _ in zip(self._chain(tokens), kv_blocks):
            node = node.children.setdefault(blk, _RadixNode())
            node.block_hash = h
        return new

    def _drop(self, b: CachedBlock) -> None:
        super()._drop(b)        # the trie keeps the edge; a dangling hash reads as a miss and is overwritten on re-insert

    def clear(self) -> None:
        super().clear()
        self.root = _RadixNode()
