"""Window batching of incoming requests and copy-on-write sharing of prompt KV between requests.

``RequestBatcher`` collects requests submitted from coroutine handlers and hands them to a worker in batches: a batch is
released when ``max_batch_size`` requests wait, or ``min_batch_size`` wait, or the oldest has waited ``max_wait_ms``.
The continuous-batching engine (``engine/engine.py``) supersedes it for token-level scheduling; the batcher serves
front ends that want request-level batches (embedding-style calls, the mock model, the perplexity endpoint).

``KVCacheSharing`` tracks which sequences share the cache blocks of a common prompt: a region is created for the first
request with that prompt, later requests attach (reference counts go up, nothing is copied), and the first write into a
shared block copies it (``PagedKVCache.fork`` + the allocator's copy-on-write do the block work).

Parity: reference ``metal_marlin/serving/mmfp4_server.py:72-330`` (``KVCacheSharing``: ``create_region``, ``attach``,
``write``/COW, ``release``, stats) and ``:590-720`` (``BatchConfig``, ``BatchedRequest``, ``RequestBatcher.submit`` /
``get_batch`` / ``complete_batch``).
"""
from __future__ import annotations

import asyncio
import hashlib
import time
import uuid
from collections import deque
from dataclasses import dataclass, field
from typing import Any, Deque, Dict, List, Optional, Sequence

from ..kv.paged import PagedKVCache


@dataclass
class BatchConfig:
    max_batch_size: int = 32
    min_batch_size: int = 1
    max_wait_ms: float = 10.0


@dataclass
class BatchedRequest:
    request: Any
    future: "asyncio.Future"
    arrival: float = field(default_factory=time.monotonic)
    request_id: str = field(default_factory=lambda: uuid.uuid4().hex)


class RequestBatcher:
    def __init__(self, config: Optional[BatchConfig] = None):
        self.config = config or BatchConfig()
        self._queue: Deque[BatchedRequest] = deque()
        self._event = asyncio.Event()
        self._pending: Dict[str, List[BatchedRequest]] = {}
        self.batches_formed = 0
        self.requests_seen = 0

    async def submit(self, request: Any) -> "asyncio.Future":
        """Queue a request; the returned future resolves with its result when its batch completes."""
        fut = asyncio.get_running_loop().create_future()
        self._queue.append(BatchedRequest(request, fut))
        self.requests_seen += 1
        self._event.set()
        return fut

    async def get_batch(self) -> List[BatchedRequest]:
        """Waits until the release rule fires, then returns up to ``max_batch_size`` requests (oldest first)."""
        c = self.config
        while True:
            if not self._queue:
                self._event.clear()
                await self._event.wait()
                continue
            waited_ms = (time.monotonic() - self._queue[0].arrival) * 1e3
            if len(self._queue) >= c.max_batch_size or (len(self._queue) >= c.min_batch_size and waited_ms >= c.max_wait_ms) \
                    or waited_ms >= 4 * c.max_wait_ms:
                break
            self._event.clear()
            try:
                await asyncio.wait_for(self._event.wait(), timeout=max(1e-4, (c.max_wait_ms - waited_ms) / 1e3))
            except asyncio.TimeoutError:
                pass
        batch = [self._queue.popleft() for _ in range(min(c.max_batch_size, len(self._queue)))]
        self._pending[batch[0].request_id] = batch
        self.batches_formed += 1
        return batch

    def complete_batch(self, batch: Sequence[BatchedRequest], results: Sequence[Any]) -> None:
        for br, res in zip(batch, results):
            if not br.future.done():
                if isinstance(res, BaseException):
                    br.future.set_exception(res)
                else:
                    br.future.set_result(res)
        self._pending.pop(batch[0].request_id, None)

    def fail_batch(self, batch: Sequence[BatchedRequest], exc: BaseException) -> None:
        self.complete_batch(batch, [exc] * len(batch))

    @property
    def queue_depth(self) -> int:
        return len(self._queue)


# -----------------------------------------------------------------------------------------------------------------
@dataclass
class SharedRegion:
    region_id: str
    owner: Any                      # sequence id whose blocks hold the prompt
    num_tokens: int
    members: List[Any] = field(default_factory=list)
    created: float = field(default_factory=time.monotonic)


class KVCacheSharing:
    """Prompt sharing on top of :class:`PagedKVCache`: requests with an identical prompt attach to one region instead of
    recomputing (and re-storing) its KV; blocks are copied only when a member writes into a shared block."""

    def __init__(self, cache: PagedKVCache):
        self.cache = cache
        self.regions: Dict[str, SharedRegion] = {}
        self._by_seq: Dict[Any, str] = {}
        self.attached = 0
        self.tokens_saved = 0

    @staticmethod
    def prompt_key(tokens: Sequence[int]) -> str:
        return hashlib.blake2b(b",".join(str(int(t)).encode() for t in tokens), digest_size=16).hexdigest()

    def create_region(self, sid, tokens: Sequence[int]) -> SharedRegion:
        """Admit ``sid`` with its prompt and publish the prompt as a shareable region (the caller runs the prompt pass)."""
        key = self.prompt_key(tokens)
        if not self.cache.table.has(sid):
            self.cache.admit(sid, tokens)
        reg = SharedRegion(key, sid, len(tokens), [sid])
        self.regions[key] = reg
        self._by_seq[sid] = key
        return reg

    def attach(self, sid, tokens: Sequence[int]) -> Optional[SharedRegion]:
        """Share the blocks of an existing region with ``sid`` (no prompt pass needed); None if no region matches."""
        reg = self.regions.get(self.prompt_key(tokens))
        if reg is None or not self.cache.table.has(reg.owner):
            return None
        self.cache.fork(reg.owner, sid)
        reg.members.append(sid)
        self._by_seq[sid] = reg.region_id
        self.attached += 1
        self.tokens_saved += reg.num_tokens
        return reg

    def append(self, sid, n: int = 1) -> List[int]:
        """Slots for ``n`` new tokens of ``sid``; a shared last block is copied first (copy-on-write)."""
        return self.cache.append(sid, n)

    def release(self, sid) -> None:
        key = self._by_seq.pop(sid, None)
        if key is not None and key in self.regions:
            reg = self.regions[key]
            if sid in reg.members:
                reg.members.remove(sid)
            if not reg.members:
                del self.regions[key]
            elif reg.owner == sid:
                reg.owner = reg.members[0]
        self.cache.release(sid)

    def stats(self) -> Dict[str, Any]:
        return {"regions": len(self.regions), "attached": self.attached, "tokens_saved": self.tokens_saved,
                "members": sum(len(r.members) for r in self.regions.values())}
