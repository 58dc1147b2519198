"""Host-side bookkeeping of the paged KV cache: block allocator, page tables, eviction and
prompt-prefix sharing.  The device pools live in ``models.transformer.PagedKVStorage``; this module
only hands out block ids, so it is identical for MLA latent caches and GQA K/V caches.

Parity: reference ``metal_marlin/paged/allocator.py:175`` (``BlockAllocator``: free list, refcounts,
copy-on-write ``:422``, contiguous best-fit runs ``:250-385``, fragmentation metric),
``metal_marlin/paged/page_table.py:33`` (``PageTable``: add / append / fork / cow / slot mapping),
``metal_marlin/paged/cache_manager.py:154`` (``PagedKVCache``: eviction LRU/LFU/weighted, TTL,
prompt-hash sharing, fork), ``metal_marlin/paged/mla_cache.py:534`` (prefix-hash block reuse),
``metal_marlin/paged/allocator.py:516`` (``MultimodalBlockAllocator``).
"""
from __future__ import annotations

import enum
import hashlib
import time
from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Callable, Dict, Iterable, List, Optional, Sequence, Tuple


class OutOfBlocks(RuntimeError):
    pass


class BlockAllocator:
    """Fixed pool of ``num_blocks`` blocks with reference counts."""

    def __init__(self, num_blocks: int, block_size: int = 16):
        self.num_blocks, self.block_size = num_blocks, block_size
        self._free: List[int] = list(range(num_blocks - 1, -1, -1))     # pop() gives the lowest id
        self._free_set = set(self._free)
        self._ref = [0] * num_blocks
        self.cow_copies = 0

    # ------------------------------------------------------------------ basic
    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_allocated(self) -> int:
        return self.num_blocks - len(self._free)

    def can_allocate(self, n: int) -> bool:
        return len(self._free) >= n

    def allocate(self) -> int:
        if not self._free:
            raise OutOfBlocks("no free KV blocks")
        b = self._free.pop()
        self._free_set.discard(b)
        self._ref[b] = 1
        return b

    def allocate_many(self, n: int) -> List[int]:
        if len(self._free) < n:
            raise OutOfBlocks(f"need {n} blocks, {len(self._free)} free")
        return [self.allocate() for _ in range(n)]

    def allocate_contiguous(self, n: int) -> List[int]:
        """Best-fit run of ``n`` consecutive block ids (smallest free run that fits)."""
        if n <= 0:
            return []
        runs = self.free_runs()
        fit = [(length, start) for start, length in runs if length >= n]
        if not fit:
            raise OutOfBlocks(f"no contiguous run of {n} blocks")
        _, start = min(fit)
        ids = list(range(start, start + n))
        taken = set(ids)
        self._free = [b for b in self._free if b not in taken]
        self._free_set -= taken
        for b in ids:
            self._ref[b] = 1
        return ids

    def free_runs(self) -> List[Tuple[int, int]]:
        ids = sorted(self._free_set)
        runs, i = [], 0
        while i < len(ids):
            j = i
            while j + 1 < len(ids) and ids[j + 1] == ids[j] + 1:
                j += 1
            runs.append((ids[i], j - i + 1))
            i = j + 1
        return runs

    def fragmentation(self) -> float:
        """1 - largest free run / free blocks (0 = one contiguous hole)."""
        if not self._free:
            return 0.0
        return 1.0 - max(length for _, length in self.free_runs()) / len(self._free)

    def ref_count(self, b: int) -> int:
        return self._ref[b]

    def incref(self, b: int) -> None:
        assert self._ref[b] > 0, "incref on a free block"
        self._ref[b] += 1

    def free(self, b: int) -> None:
        assert self._ref[b] > 0, f"double free of block {b}"
        self._ref[b] -= 1
        if self._ref[b] == 0:
            self._free.append(b)
            self._free_set.add(b)

    def free_many(self, blocks: Iterable[int]) -> None:
        for b in blocks:
            self.free(b)

    def cow(self, b: int, copy_fn: Optional[Callable[[int, int], None]] = None) -> int:
        """Copy-on-write: a block shared by several sequences is duplicated before it is written.
        Returns the block the caller may write (``b`` itself when it is not shared)."""
        if self._ref[b] <= 1:
            return b
        nb = self.allocate()
        if copy_fn is not None:
            copy_fn(b, nb)
        self._ref[b] -= 1
        self.cow_copies += 1
        return nb

    def usage(self) -> float:
        return self.num_allocated / max(1, self.num_blocks)

    def needs_compaction(self, max_fragmentation: float = 0.75, max_runs: int = 32) -> bool:
        """The free space is split so badly that contiguous requests suffer (parity: the reference compacts above a
        fragmentation of 0.75 or more than 32 free runs)."""
        return self.fragmentation() > max_fragmentation or len(self.free_runs()) > max_runs

    def compaction_plan(self) -> List[Tuple[int, int]]:
        """Moves ``(src, dst)`` that pack the allocated blocks into the lowest ids: the highest allocated block goes into
        the lowest hole until no hole lies below an allocated block.  Apply with :meth:`apply_moves`."""
        holes = sorted(self._free_set)
        used = sorted((b for b in range(self.num_blocks) if self._ref[b] > 0), reverse=True)
        moves = []
        for src, dst in zip(used, holes):
            if dst >= src:
                break
            moves.append((src, dst))
        return moves

    def apply_moves(self, moves: Sequence[Tuple[int, int]]) -> None:
        """Book-keeping of a compaction: reference counts follow the blocks, the free list is rebuilt."""
        for src, dst in moves:
            assert self._ref[dst] == 0 and self._ref[src] > 0
            self._ref[dst], self._ref[src] = self._ref[src], 0
        self._free = [b for b in range(self.num_blocks - 1, -1, -1) if self._ref[b] == 0]
        self._free_set = set(self._free)


class MultimodalBlockAllocator(BlockAllocator):
    """Block allocator with a reserved region for vision-encoder tokens (image blocks are
    immutable and shareable between requests that reference the same image)."""

    def __init__(self, num_blocks: int, block_size: int = 16, vision_fraction: float = 0.25):
        super().__init__(num_blocks, block_size)
        self.vision_budget = int(num_blocks * vision_fraction)
        self.vision_blocks: Dict[str, List[int]] = {}
        self._vision_used = 0

    def allocate_image(self, image_hash: str, n_tokens: int) -> List[int]:
        if image_hash in self.vision_blocks:
            for b in self.vision_blocks[image_hash]:
                self.incref(b)
            return self.vision_blocks[image_hash]
        n = -(-n_tokens // self.block_size)
        if self._vision_used + n > self.vision_budget:
            raise OutOfBlocks("vision block budget exhausted")
        ids = self.allocate_many(n)
        self.vision_blocks[image_hash] = ids
        self._vision_used += n
        return ids

    def release_image(self, image_hash: str) -> None:
        ids = self.vision_blocks.get(image_hash)
        if not ids:
            return
        self.free_many(ids)
        if self.ref_count(ids[0]) == 0:
            self._vision_used -= len(ids)
            del self.vision_blocks[image_hash]


@dataclass
class SequenceEntry:
    blocks: List[int] = field(default_factory=list)
    num_tokens: int = 0


class PageTable:
    """Maps sequence ids to block lists."""

    def __init__(self, allocator: BlockAllocator):
        self.alloc = allocator
        self.block_size = allocator.block_size
        self.seqs: Dict[object, SequenceEntry] = {}

    def has(self, sid) -> bool:
        return sid in self.seqs

    def add_sequence(self, sid, num_tokens: int = 0, blocks: Optional[List[int]] = None) -> List[int]:
        assert sid not in self.seqs, f"sequence {sid!r} exists"
        ent = SequenceEntry(list(blocks or []), 0)
        self.seqs[sid] = ent
        if blocks:
            ent.num_tokens = min(num_tokens, len(blocks) * self.block_size)
        self.reserve(sid, num_tokens)
        ent.num_tokens = num_tokens
        return ent.blocks

    def blocks_needed(self, sid, new_total_tokens: int) -> int:
        have = len(self.seqs[sid].blocks) if sid in self.seqs else 0
        return max(0, -(-new_total_tokens // self.block_size) - have)

    def reserve(self, sid, total_tokens: int) -> List[int]:
        """Ensure capacity for ``total_tokens`` tokens; returns newly allocated blocks."""
        ent = self.seqs[sid]
        need = self.blocks_needed(sid, total_tokens)
        new = self.alloc.allocate_many(need) if need else []
        ent.blocks.extend(new)
        return new

    def append_tokens(self, sid, n: int = 1, copy_fn=None) -> List[int]:
        """Account for ``n`` new tokens; allocates blocks as needed and un-shares the block that will
        be written (copy-on-write).  Returns the slot ids of the new tokens."""
        ent = self.seqs[sid]
        start = ent.num_tokens
        self.reserve(sid, start + n)
        slots = []
        for t in range(start, start + n):
            bi = t // self.block_size
            b = ent.blocks[bi]
            if self.alloc.ref_count(b) > 1:
                ent.blocks[bi] = b = self.alloc.cow(b, copy_fn)
            slots.append(b * self.block_size + t % self.block_size)
        ent.num_tokens = start + n
        return slots

    def slot_mapping(self, sid, start: int, n: int) -> List[int]:
        ent = self.seqs[sid]
        bs = self.block_size
        return [ent.blocks[t // bs] * bs + t % bs for t in range(start, start + n)]

    def block_table(self, sid) -> List[int]:
        return self.seqs[sid].blocks

    def num_tokens(self, sid) -> int:
        return self.seqs[sid].num_tokens

    def fork(self, parent, child) -> None:
        """Child shares every block of the parent (beam search / n > 1 sampling / prompt sharing)."""
        p = self.seqs[parent]
        for b in p.blocks:
            self.alloc.incref(b)
        self.seqs[child] = SequenceEntry(list(p.blocks), p.num_tokens)

    def truncate(self, sid, num_tokens: int) -> None:
        """Drop tokens beyond ``num_tokens`` (speculative-decoding rollback); frees whole blocks."""
        ent = self.seqs[sid]
        keep = -(-num_tokens // self.block_size)
        for b in ent.blocks[keep:]:
            self.alloc.free(b)
        del ent.blocks[keep:]
        ent.num_tokens = min(ent.num_tokens, num_tokens)

    def remove(self, sid) -> None:
        ent = self.seqs.pop(sid, None)
        if ent:
            self.alloc.free_many(ent.blocks)

    def padded_tables(self, sids: Sequence, pad: int = 0) -> List[List[int]]:
        width = max((len(self.seqs[s].blocks) for s in sids), default=0)
        return [self.seqs[s].blocks + [pad] * (width - len(self.seqs[s].blocks)) for s in sids]


class EvictionPolicy(enum.Enum):
    LRU = "lru"
    LFU = "lfu"
    WEIGHTED = "weighted"    # age / (1 + hits)
    FIFO = "fifo"            # oldest insertion first
    ADAPTIVE = "adaptive"    # recency when the cache rarely hits, frequency when it hits often (weights follow the hit rate)


def hash_tokens(tokens: Sequence[int], parent: str = "") -> str:
    h = hashlib.blake2b(digest_size=16)
    h.update(parent.encode())
    h.update(b",".join(str(int(t)).encode() for t in tokens))
    return h.hexdigest()


@dataclass
class _CachedBlock:
    block: int
    hits: int = 0
    last_used: float = 0.0
    created: float = 0.0


class PrefixCache:
    """Block-granular prompt prefix cache: a chain hash of each *full* block of tokens maps to the
    block that already holds its KV.  Cached blocks hold one reference of their own; eviction
    releases it.  Parity: reference ``metal_marlin/serving/scheduler.py:80`` and
    ``metal_marlin/paged/cache_manager.py`` prompt-hash sharing."""

    def __init__(self, allocator: BlockAllocator, max_blocks: Optional[int] = None,
                 policy: EvictionPolicy = EvictionPolicy.LRU, ttl_s: Optional[float] = None):
        self.alloc = allocator
        self.block_size = allocator.block_size
        self.max_blocks = max_blocks if max_blocks is not None else allocator.num_blocks // 2
        self.policy, self.ttl_s = policy, ttl_s
        self.table: "OrderedDict[str, _CachedBlock]" = OrderedDict()
        self.hits = self.misses = self.evictions = 0

    def _chain(self, tokens: Sequence[int]) -> List[str]:
        out, parent = [], ""
        for i in range(0, len(tokens) - len(tokens) % self.block_size, self.block_size):
            parent = hash_tokens(tokens[i:i + self.block_size], parent)
            out.append(parent)
        return out

    def match(self, tokens: Sequence[int]) -> List[int]:
        """Longest cached prefix.  Returned blocks are inc-ref'ed for the caller."""
        now = time.monotonic()
        blocks = []
        for h in self._chain(tokens):
            cb = self.table.get(h)
            if cb is None or (self.ttl_s is not None and now - cb.created > self.ttl_s):
                break
            cb.hits += 1
            cb.last_used = now
            self.table.move_to_end(h)
            self.alloc.incref(cb.block)
            blocks.append(cb.block)
        if blocks:
            self.hits += 1
        else:
            self.misses += 1
        return blocks

    def insert(self, tokens: Sequence[int], blocks: Sequence[int]) -> int:
        """Register the full blocks of a prefilled prompt.  Returns how many were newly cached."""
        now = time.monotonic()
        added = 0
        for h, b in zip(self._chain(tokens), blocks):
            if h in self.table:
                continue
            while len(self.table) >= self.max_blocks:
                if not self.evict_one():
                    return added
            self.alloc.incref(b)
            self.table[h] = _CachedBlock(b, 0, now, now)
            added += 1
        return added

    def evict_one(self) -> bool:
        if not self.table:
            return False
        now = time.monotonic()
        if self.policy is EvictionPolicy.LRU:
            key = next(iter(self.table))
        elif self.policy is EvictionPolicy.LFU:
            key = min(self.table, key=lambda k: (self.table[k].hits, self.table[k].last_used))
        elif self.policy is EvictionPolicy.FIFO:
            key = min(self.table, key=lambda k: self.table[k].created)
        elif self.policy is EvictionPolicy.ADAPTIVE:
            rate = self.hits / max(1, self.hits + self.misses)
            oldest = max(now - cb.last_used for cb in self.table.values()) or 1.0
            most = max(cb.hits for cb in self.table.values()) or 1
            key = max(self.table, key=lambda k: (1.0 - rate) * (now - self.table[k].last_used) / oldest
                      - rate * self.table[k].hits / most)
        else:
            key = max(self.table, key=lambda k: (now - self.table[k].last_used) / (1 + self.table[k].hits))
        cb = self.table.pop(key)
        self.alloc.free(cb.block)
        self.evictions += 1
        return True

    def evict_batch(self, n: int) -> int:
        """Evict up to ``n`` cached blocks in one go; returns how many went."""
        done = 0
        while done < n and self.evict_one():
            done += 1
        return done

    def proactive_evict(self, pressure: float = 0.9) -> int:
        """While more than ``pressure`` of the allocator's blocks are in use, release cached blocks (the ones no sequence
        holds any more become free), so that admissions do not have to evict one block at a time under load."""
        n = 0
        while self.alloc.usage() > pressure and self.evict_one():
            n += 1
        return n

    def evict_until(self, n_free: int) -> int:
        """Evict cached blocks until the allocator has ``n_free`` free blocks (or the cache is empty)."""
        n = 0
        while self.alloc.num_free < n_free and self.evict_one():
            n += 1
        return n

    def stats(self) -> dict:
        return {"entries": len(self.table), "hits": self.hits, "misses": self.misses, "evictions": self.evictions}


class PagedKVCache:
    """Allocator + page table + prefix cache behind one object (what schedulers talk to)."""

    def __init__(self, num_blocks: int, block_size: int = 16, enable_prefix_cache: bool = True,
                 policy: EvictionPolicy = EvictionPolicy.LRU, copy_fn=None):
        self.alloc = BlockAllocator(num_blocks, block_size)
        self.table = PageTable(self.alloc)
        self.prefix = PrefixCache(self.alloc, policy=policy) if enable_prefix_cache else None
        self.block_size = block_size
        self.copy_fn = copy_fn

    def can_admit(self, n_tokens: int, reserve_blocks: int = 0) -> bool:
        need = -(-n_tokens // self.block_size) + reserve_blocks
        if self.alloc.num_free >= need:
            return True
        if self.prefix is not None:
            self.prefix.evict_until(need)
        return self.alloc.num_free >= need

    def admit(self, sid, tokens: Sequence[int]) -> int:
        """Create a sequence for ``tokens``; returns the number of tokens whose KV is already cached."""
        shared = self.prefix.match(tokens) if self.prefix is not None else []
        # never reuse the block containing the last prompt token: its logits must be recomputed
        max_shared = (len(tokens) - 1) // self.block_size
        for b in shared[max_shared:]:
            self.alloc.free(b)
        shared = shared[:max_shared]
        cached = len(shared) * self.block_size
        try:
            self.table.add_sequence(sid, len(tokens), blocks=shared)
        except OutOfBlocks:
            self.table.seqs.pop(sid, None)
            self.alloc.free_many(shared)
            raise
        return cached

    def publish(self, sid, tokens: Sequence[int]) -> None:
        if self.prefix is not None:
            self.prefix.insert(tokens, self.table.block_table(sid))

    def append(self, sid, n: int = 1) -> List[int]:
        if not self.can_admit(0, reserve_blocks=self.table.blocks_needed(sid, self.table.num_tokens(sid) + n)):
            raise OutOfBlocks("cannot extend sequence")
        return self.table.append_tokens(sid, n, self.copy_fn)

    def fork(self, parent, child) -> None:
        self.table.fork(parent, child)

    def release(self, sid) -> None:
        self.table.remove(sid)

    def compact(self, copy_fn=None, force: bool = False) -> int:
        """Pack the blocks in use into the lowest ids when the allocator asks for it (or ``force``): every moved block is
        copied with ``copy_fn(src, dst)`` (default: the cache's own copy function) and every page table and prefix-cache
        entry that named it is rewritten.  Returns the number of blocks moved.  Call between iterations only."""
        if not force and not self.alloc.needs_compaction():
            return 0
        moves = self.alloc.compaction_plan()
        if not moves:
            return 0
        copy_fn = copy_fn or self.copy_fn
        remap = dict(moves)
        for src, dst in moves:
            if copy_fn is not None:
                copy_fn(src, dst)
        self.alloc.apply_moves(moves)
        for ent in self.table.seqs.values():
            ent.blocks[:] = [remap.get(b, b) for b in ent.blocks]
        if self.prefix is not None:
            for cb in self.prefix.table.values():
                cb.block = remap.get(cb.block, cb.block)
        return len(moves)

    def stats(self) -> dict:
        s = {"blocks": self.alloc.num_blocks, "free": self.alloc.num_free, "usage": self.alloc.usage(),
             "fragmentation": self.alloc.fragmentation(), "cow_copies": self.alloc.cow_copies,
             "sequences": len(self.table.seqs)}
        if self.prefix is not None:
            s["prefix"] = self.prefix.stats()
        return s
