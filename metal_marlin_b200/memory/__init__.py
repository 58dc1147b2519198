"""Memory runtime: arenas over caller-owned slabs (device / pinned / symmetric), a step-scoped bump allocator, pinned
staging pools, asynchronous weight streaming, an LRU expert cache and a memory-pressure monitor.

Parity: reference ``metal_marlin/memory/*`` (buffer pools / recycler / rings / heap allocator, mmap weight manager,
zero-copy transfer manager, memory-pressure monitor, CUDA pinned pool and transfer stream), ``_buffer_pool.py``,
``buffer_ring.py``, ``heap_allocator.py``, ``workspace_buffer.py``, ``expert_cache.py`` and ``cpp/src/pool.cpp``.  The
allocator bookkeeping is native (``csrc/runtime.cpp``); tensors handed out are views into one slab, so nothing on the
request path calls ``cudaMalloc``.
"""
from .arena import Arena, BumpAllocator, WorkspaceBuffer
from .expert_cache import ExpertCache, ExpertWeightStreamer, TileCoordinator
from .model_memory import (CompactionConfig, CompactionStats, CUDAPinnedPool, ExpertMetadata, LayerMetadata, MemoryCompactor, MemoryStats,
                           MLACompressionRatio, MMAPWeightConfig, MMAPWeightManager, MMAPWeightStats, MMFP4MemoryManager, PooledBuffer)
from .pressure import MemoryPressureMonitor, PressureLevel
from .pools import (BufferPool, BufferPoolStats, RingBuffer, TransferStream, TransientBuffer, TransientBufferCPP, get_ring_buffer,
                    get_transient_buffer_cpp, reset_ring_buffer, reset_transient_buffer_cpp, transient_buffer_cpp_stats)
from .streaming import PinnedPool, WeightStreamer

__all__ = ["Arena", "BumpAllocator", "WorkspaceBuffer", "ExpertCache", "ExpertWeightStreamer", "TileCoordinator", "MemoryPressureMonitor", "PressureLevel", "PinnedPool",
           "WeightStreamer", "BufferPool", "BufferPoolStats", "RingBuffer", "TransferStream", "get_ring_buffer", "reset_ring_buffer", "CompactionConfig",
           "CompactionStats", "CUDAPinnedPool", "ExpertMetadata", "LayerMetadata", "MemoryCompactor", "MemoryStats", "MLACompressionRatio",
           "MMAPWeightConfig", "MMAPWeightManager", "MMAPWeightStats", "MMFP4MemoryManager", "PooledBuffer", "TransientBuffer", "TransientBufferCPP",
           "get_transient_buffer_cpp", "reset_transient_buffer_cpp", "transient_buffer_cpp_stats"]
