"""KV caches: the paged pool (allocator, page table, prefix caches, eviction), contiguous and quantized caches, tiered
and radix prompt caches, and helpers to run and validate attention over pages.

The names of the reference's ``metal_marlin.paged`` and ``metal_marlin.cache`` packages are available here (parity:
``paged/__init__.py``: ``KVBlock`` / ``KVBlockConfig`` / ``BlockState``, ``MLABlock*`` / ``MLACacheConfig``, ``EvictionPolicy`` /
``CacheStats``, ``paged_attention`` / ``paged_attention_v1`` / ``mla_attention`` / ``write_kv_to_blocks``, the parity validators;
``cache/__init__.py``: ``PrefixMatch``, ``CachedBlock``, ``CacheMetrics``, ``QuantizedKVCache``, ``compress_kv`` / ``decompress_kv``,
``hash_prefix`` / ``hash_tokens``)."""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .contiguous import CacheConfig, KVCache, MLAKVCache, PersistentKVCache, dequantize_kv, quantize_kv
from .paged import (BlockAllocator, EvictionPolicy, MultimodalBlockAllocator, OutOfBlocks, PagedKVCache, PageTable, PrefixCache,
                    SequenceEntry, hash_tokens)
from .prompt_cache import (CachedBlock, CacheMetrics, PrefixCacheConfig, PrefixMatch, RadixPrefixCache, StorageTier, TieredPrefixCache)

hash_prefix = hash_tokens
compress_kv = quantize_kv
decompress_kv = dequantize_kv
MLABlockAllocator = BlockAllocator            # a latent row is one "head" of width kv_lora_rank + rope_dim
SequenceState = SequenceEntry


class BlockState(enum.Enum):
    FREE = "free"
    ALLOCATED = "allocated"
    SHARED = "shared"                          # more than one reference (forked sequences, cached prefixes)


MLABlockState = BlockState
MultimodalBlockState = BlockState


class ScalingStrategy(enum.Enum):
    PER_TENSOR = "tensor"
    PER_TOKEN = "token"
    PER_GROUP = "group"


class TokenModality(enum.Enum):
    TEXT = "text"
    IMAGE = "image"


SequenceModality = TokenModality


@dataclass
class KVBlockConfig:
    block_size: int = 16
    num_kv_heads: int = 8
    head_dim: int = 128
    dtype: str = "bf16"                        # bf16 | fp8 | int8 | fp4 | int4

    @property
    def bytes_per_token(self) -> float:
        per = {"bf16": 2.0, "fp16": 2.0, "fp8": 1.0, "int8": 1.0, "fp4": 0.5, "int4": 0.5}[self.dtype]
        scale = 0.0 if self.dtype in ("bf16", "fp16") else 4.0 * self.num_kv_heads           # one fp32 scale per row and head
        return 2 * (self.num_kv_heads * self.head_dim * per + scale)

    @property
    def bytes_per_block(self) -> float:
        return self.bytes_per_token * self.block_size


@dataclass
class MLACacheConfig:
    block_size: int = 16
    kv_lora_rank: int = 512
    rope_dim: int = 64
    dtype: str = "bf16"

    @property
    def bytes_per_token(self) -> float:
        per = {"bf16": 2.0, "fp16": 2.0, "fp8": 1.0, "int8": 1.0, "fp4": 0.5, "int4": 0.5}[self.dtype]
        return (self.kv_lora_rank + self.rope_dim) * per + (0.0 if self.dtype in ("bf16", "fp16") else 4.0)


@dataclass
class KVBlock:
    """One block of the pool as the allocator sees it."""
    block_id: int
    ref_count: int = 0
    num_tokens: int = 0

    @property
    def state(self) -> BlockState:
        return BlockState.FREE if self.ref_count == 0 else (BlockState.SHARED if self.ref_count > 1 else BlockState.ALLOCATED)

    @classmethod
    def of(cls, allocator: BlockAllocator, block_id: int) -> "KVBlock":
        return cls(block_id, allocator.ref_count(block_id))


MLABlock = KVBlock


@dataclass
class ImageRegion:
    image_hash: str
    blocks: List[int]
    num_tokens: int


@dataclass
class CacheStats:
    blocks: int
    free: int
    usage: float
    fragmentation: float
    sequences: int
    cow_copies: int = 0
    prefix_hits: int = 0
    prefix_misses: int = 0
    evictions: int = 0

    @classmethod
    def of(cls, cache: PagedKVCache) -> "CacheStats":
        s = cache.stats()
        p = s.get("prefix", {})
        return cls(s["blocks"], s["free"], s["usage"], s["fragmentation"], s["sequences"], s.get("cow_copies", 0), p.get("hits", 0),
                   p.get("misses", 0), p.get("evictions", 0))


EvictionStats = CacheStats


@dataclass
class SequenceEvictionMetadata:
    sequence_id: object
    num_blocks: int
    last_used: float = 0.0
    hits: int = 0


class QuantizedKVCache(KVCache):
    """Contiguous cache with quantized storage (``fp8`` by default; ``int8`` / ``fp4`` / ``fp8_e5m2`` too)."""

    def __init__(self, num_layers: int, batch: int, num_kv_heads: int, head_dim: int, max_seq_len: int, dtype: str = "fp8", device="cpu", **kw):
        super().__init__(CacheConfig(num_layers=num_layers, num_kv_heads=num_kv_heads, head_dim=head_dim, max_seq_len=max_seq_len,
                                     batch_size=batch, dtype=dtype, **kw), device)


class QuantizedKVCacheFP4Int8(QuantizedKVCache):
    """Keys in FP4, values in INT8 is what the reference's class of this name stores; one storage mode per cache here: FP4."""

    def __init__(self, *a, **kw):
        kw.setdefault("dtype", "fp4")
        super().__init__(*a, **kw)


# ------------------------------------------------------------------------------------------------ attention over pages
def write_kv_to_blocks(k_pool, v_pool, k: torch.Tensor, v: Optional[torch.Tensor], slots: torch.Tensor) -> None:
    """Rows ``k, v [n, Hkv, D]`` into cache rows ``slots [n]`` of bf16 or quantized pools."""
    from .. import ops
    slots = slots.to(torch.int64)
    for pool, rows in ((k_pool, k), (v_pool, v)):
        if pool is None or rows is None:
            continue
        if isinstance(pool, ops.FP8KV):
            pool.store(slots, rows.reshape(rows.shape[0], *pool.shape[1:]))
        else:
            pool.view(pool.shape[0], -1).index_copy_(0, slots, rows.reshape(rows.shape[0], -1).to(pool.dtype))


def paged_attention(q: torch.Tensor, k_pool, v_pool, block_tables: torch.Tensor, ctx_lens: torch.Tensor, *, scale: Optional[float] = None,
                    block_size: int = 16, window: int = 0) -> torch.Tensor:
    """Decode attention ``q [B, Hq, D]`` over paged keys / values ``[slots, Hkv, D]``."""
    from .. import ops
    B, Hq, D = q.shape
    Hkv = k_pool.shape[1]
    return ops.paged_attention(q, k_pool, v_pool, block_tables, ctx_lens, Hq=Hq, Hkv=Hkv, dqk=D, dv=v_pool.shape[-1], block_size=block_size,
                               scale=scale if scale is not None else D ** -0.5, window=window)


paged_attention_v1 = paged_attention


def mla_attention(q_lat: torch.Tensor, latent_pool, block_tables: torch.Tensor, ctx_lens: torch.Tensor, kv_lora_rank: int, *,
                  scale: float, block_size: int = 16) -> torch.Tensor:
    """Absorbed MLA decode: ``q_lat [B, H, R + dr]`` against latent rows ``[slots, R + dr]``; returns ``[B, H, R]``."""
    from .. import ops
    B, H, W = q_lat.shape
    return ops.paged_attention(q_lat, latent_pool, None, block_tables, ctx_lens, Hq=H, Hkv=1, dqk=W, dv=kv_lora_rank, block_size=block_size,
                               scale=scale)


def compute_linear_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: Optional[float] = None) -> torch.Tensor:
    """Plain attention over contiguous (linear, un-paged) keys: ``q [B, Hq, D]``, ``k, v [B, N, Hkv, D]`` -> ``[B, Hq, D]``."""
    B, Hq, D = q.shape
    g = Hq // k.shape[2]
    kk, vv = k.float().repeat_interleave(g, 2), v.float().repeat_interleave(g, 2)
    s = torch.einsum("bhd,bnhd->bhn", q.float(), kk) * (scale if scale is not None else D ** -0.5)
    return torch.einsum("bhn,bnhd->bhd", torch.softmax(s, -1), vv)


@dataclass
class ParityConfig:
    batch: int = 2
    num_heads: int = 4
    num_kv_heads: int = 2
    head_dim: int = 64
    seq_len: int = 70
    block_size: int = 16
    tolerance: float = 2e-2
    seed: int = 0
    device: str = "cpu"


ValidationConfig = ParityConfig


@dataclass
class ParityResult:
    passed: bool
    max_abs_error: float
    tolerance: float
    details: Dict[str, float] = field(default_factory=dict)


ParityValidationResult = ParityResult


def validate_paged_v1_parity(config: Optional[ParityConfig] = None) -> ParityResult:
    """Random keys / values written into shuffled pages, attention over the pages against attention over the same rows
    laid out contiguously."""
    c = config or ParityConfig()
    g = torch.Generator().manual_seed(c.seed)
    dev = torch.device(c.device)
    nb_seq = -(-c.seq_len // c.block_size)
    perm = torch.randperm(c.batch * nb_seq, generator=g)
    bt = perm.view(c.batch, nb_seq).to(torch.int32).to(dev)
    k = torch.randn(c.batch, c.seq_len, c.num_kv_heads, c.head_dim, generator=g).to(torch.bfloat16).to(dev)
    v = torch.randn(c.batch, c.seq_len, c.num_kv_heads, c.head_dim, generator=g).to(torch.bfloat16).to(dev)
    q = torch.randn(c.batch, c.num_heads, c.head_dim, generator=g).to(torch.bfloat16).to(dev)
    kp = torch.zeros(c.batch * nb_seq * c.block_size, c.num_kv_heads, c.head_dim, dtype=torch.bfloat16, device=dev)
    vp = torch.zeros_like(kp)
    tok = torch.arange(c.seq_len, device=dev)
    for b in range(c.batch):
        slots = bt[b, tok // c.block_size].long() * c.block_size + tok % c.block_size
        write_kv_to_blocks(kp, vp, k[b], v[b], slots)
    cl = torch.full((c.batch,), c.seq_len, dtype=torch.int32, device=dev)
    got = paged_attention(q, kp, vp, bt, cl, block_size=c.block_size).float()
    ref = compute_linear_attention(q, k, v)
    err = float((got - ref).abs().max())
    return ParityResult(err <= c.tolerance, err, c.tolerance, {"ref_abs_max": float(ref.abs().max())})


validate_parity = validate_paged_v1_parity
validate_paged_linear_parity = validate_paged_v1_parity
validate_paged_block_pool_parity = validate_paged_v1_parity
run_paged_v1_parity_test = validate_paged_v1_parity


class ParityValidator:
    def __init__(self, config: Optional[ParityConfig] = None):
        self.config = config or ParityConfig()

    def run(self) -> ParityResult:
        return validate_paged_v1_parity(self.config)


def run_comprehensive_parity_suite(device: str = "cpu") -> List[ParityResult]:
    """Several shapes: grouped and ungrouped heads, ragged last block, one-block sequences."""
    cases = [ParityConfig(device=device), ParityConfig(num_heads=8, num_kv_heads=8, head_dim=128, seq_len=33, device=device),
             ParityConfig(batch=3, num_heads=8, num_kv_heads=1, seq_len=16, device=device), ParityConfig(seq_len=5, device=device)]
    return [validate_paged_v1_parity(c) for c in cases]


def compare_memory_usage(seq_lens: Sequence[int], max_seq_len: int, block_config: Optional[KVBlockConfig] = None, num_layers: int = 1) -> Dict:
    """Bytes of a contiguous cache sized for ``max_seq_len`` per sequence against the paged pool that holds the same
    sequences (whole blocks)."""
    c = block_config or KVBlockConfig()
    contiguous = len(seq_lens) * max_seq_len * c.bytes_per_token * num_layers
    blocks = sum(-(-n // c.block_size) for n in seq_lens)
    paged = blocks * c.bytes_per_block * num_layers
    return {"contiguous_bytes": contiguous, "paged_bytes": paged, "blocks": blocks, "savings": 1.0 - paged / max(contiguous, 1.0),
            "internal_fragmentation": 1.0 - sum(seq_lens) / max(1, blocks * c.block_size)}


__all__ = [n for n in dir() if not n.startswith("_") and n not in ("annotations", "enum", "dataclass", "field", "torch", "Dict", "List",
                                                                     "Optional", "Sequence", "Tuple")]


def __getattr__(name: str):
    if name == "VisionEncoderCache":                 # content-addressed cache of encoded images (kept with the vision front end)
        from ..vision import VisionEncoderCache
        return VisionEncoderCache
    raise AttributeError(name)


__all__ += ["VisionEncoderCache"]
