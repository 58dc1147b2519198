"""Serving: OpenAI-compatible server, serving engine (mock model, formats, latency statistics), request batching and prompt
sharing, metrics, data-parallel router, terminal monitor - plus the reference's ``metal_marlin.serving`` names for the
scheduler pieces (``ContinuousSchedulerConfig``, ``IterationPlanner`` / ``IterationPlan``, ``SchedulerOutput``, ``KVCacheManager`` /
``KVRegion``, ``BatchedModelRunner``), which live in ``engine/`` and ``kv/`` here.  Resolved on first use."""
from __future__ import annotations

import importlib
from dataclasses import dataclass
from typing import List

_LAZY = {
    "ServingCppDispatcher": (".native_dispatch", "ServingCppDispatcher"), "ServingCppEngineWrapper": (".native_dispatch", "ServingCppEngineWrapper"),
    "create_serving_cpp_dispatcher": (".native_dispatch", "create_serving_cpp_dispatcher"), "DispatchHandle": (".native_dispatch", "DispatchHandle"),
    "SchedulerConfig": ("..engine.scheduler", "SchedulerConfig"), "ContinuousSchedulerConfig": ("..engine.scheduler", "SchedulerConfig"),
    "PreemptionPolicy": ("..engine.scheduler", "PreemptionPolicy"), "RequestPriority": ("..engine.request", "RequestPriority"),
    "RequestState": ("..engine.request", "RunningRequest"), "ModelConfig": ("..models.config", "ModelConfig"),
    "ServingEngine": (".engine", "ServingEngine"), "EngineConfig": (".engine", "EngineConfig"), "run_server": (".server", "run_server"),
    "app": (".server", "app"), "configure": (".server", "configure"), "MetricsCollector": (".metrics", "MetricsCollector"),
    "MoEMetrics": (".metrics", "MoEMetrics"), "PerplexityTracker": (".metrics", "PerplexityTracker"),
    "RequestBatcher": (".batching", "RequestBatcher"), "KVCacheSharing": (".batching", "KVCacheSharing"),
    "ContinuousSchedulerConfig": ("..engine.scheduler", "SchedulerConfig"), "IterationPlanner": ("..engine.scheduler", "BatchScheduler"),
    "BatchScheduler": ("..engine.scheduler", "BatchScheduler"), "FCFSScheduler": ("..engine.fcfs", "FCFSScheduler"),
    "SchedulerOutput": ("..engine.request", "SchedulerOutput"), "IterationPlan": ("..engine.request", "SchedulerOutput"),
    "GenerationRequest": ("..engine.request", "GenerationRequest"), "RequestStatus": ("..engine.request", "RequestStatus"),
    "KVCacheManager": ("..kv.paged", "PagedKVCache"), "BatchedModelRunner": ("..engine.engine", "LLMEngine"),
    "LLMEngine": ("..engine.engine", "LLMEngine"),
}


def __getattr__(name: str):
    if name in _LAZY:
        mod, attr = _LAZY[name]
        return getattr(importlib.import_module(mod, __package__), attr)
    raise AttributeError(name)


@dataclass
class KVRegion:
    """The cache rows of one sequence: its blocks and how many tokens they hold."""
    sequence_id: object
    blocks: List[int]
    num_tokens: int
    block_size: int = 16

    @classmethod
    def of(cls, cache, sequence_id) -> "KVRegion":
        return cls(sequence_id, list(cache.table.block_table(sequence_id)), cache.table.num_tokens(sequence_id), cache.block_size)

    def slots(self) -> List[int]:
        return [self.blocks[t // self.block_size] * self.block_size + t % self.block_size for t in range(self.num_tokens)]


def _kv_sharing(server=None, enable_prefix_caching: bool = True, cache=None):
    """A prompt-sharing manager over a paged cache: ``cache`` when given, else the cache of ``server`` (a serving engine), else a
    small cache of its own (stand-alone bookkeeping).  Reference ``serving/mmfp4_server.py:410``."""
    from ..kv.paged import PagedKVCache
    from .batching import KVCacheSharing
    if cache is None and server is not None:
        for holder in (server, getattr(server, "engine", None), getattr(getattr(server, "engine", None), "engine", None)):
            if isinstance(getattr(holder, "cache", None), PagedKVCache):
                cache = holder.cache
                break
    if cache is None:
        cache = PagedKVCache(num_blocks=64, block_size=16, enable_prefix_cache=enable_prefix_caching)
    return KVCacheSharing(cache)


__all__ = sorted(list(_LAZY) + ["KVRegion", "_kv_sharing"])
