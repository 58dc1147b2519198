"""Prompt-pass helpers over the paged cache: memory-aware chunked prefill with progress and timing, bulk KV writes,
a layout-friendly entry to the prompt attention kernels, and speculative prefill.

Parity: reference ``metal_marlin/inference/prefill.py`` (``PrefillConfig`` ``:97``, ``PrefillStats`` ``:124``,
``chunked_prefill`` ``:174``, ``_estimate_peak_memory`` ``:330``, ``parallel_kv_write`` ``:363``,
``flash_prefill_attention`` ``:571``, ``SpeculativePrefillConfig`` ``:777``, ``speculative_prefill`` ``:792``).  Here a chunk is
a varlen batch through ``models.mmfp4_causal_lm.prefill`` (keys and values are written by the fused norm + RoPE + scatter
kernel, attention over the cached context runs on the tcgen05 kernel), so the helpers add policy and bookkeeping, not a
second forward path.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence, Tuple

import torch

from .. import ops
from ..models.mmfp4_causal_lm import prefill as _prefill


@dataclass
class PrefillConfig:
    chunk_size: int = 4096                 # tokens per chunk; 0 = derive from free memory and ``memory_fraction``
    use_flash_attention: bool = True       # tcgen05 / mma.sync attention kernels (False: PyTorch restatement, for debugging)
    memory_fraction: float = 0.8           # share of the free device memory the activations of one chunk may take
    min_chunk: int = 256
    max_chunk: int = 32768


@dataclass
class PrefillStats:
    total_tokens: int = 0
    num_chunks: int = 0
    prefill_time_ms: float = 0.0
    tokens_per_second: float = 0.0
    peak_memory_mb: float = 0.0
    flash_attention_used: bool = False
    chunk_times_ms: List[float] = field(default_factory=list)


def estimate_chunk_bytes(cfg, chunk: int, context: int = 0) -> int:
    """Upper bound of the transient device memory of one ``chunk``-token pass: residual stream and projections in bf16,
    the widest MLP / routed-expert intermediate, fp32 logits of one row, and for MLA the per-head keys and values lifted
    from the latent cache for ``context + chunk`` positions."""
    h = cfg.hidden_size
    widest = max(2 * (cfg.intermediate_size or 0),
                 2 * (cfg.moe_intermediate_size or 0) * max(1, cfg.num_experts_per_tok + getattr(cfg, "n_shared_experts", 0)))
    attn = cfg.num_attention_heads * (cfg.dh + (getattr(cfg, "v_head_dim", 0) or cfg.dh)) + 2 * cfg.num_key_value_heads * cfg.dh
    per_tok = 2 * (4 * h + widest + attn)
    lifted = 0
    if getattr(cfg, "kv_lora_rank", 0):
        lifted = 2 * (context + chunk) * cfg.num_attention_heads * (cfg.qk_nope_head_dim + cfg.qk_rope_head_dim + cfg.v_head_dim)
    return chunk * per_tok + lifted + 4 * cfg.vocab_size


def pick_chunk_size(cfg, total_tokens: int, config: Optional[PrefillConfig] = None, free_bytes: Optional[int] = None) -> int:
    """Largest power-of-two chunk (``min_chunk``..``max_chunk``) whose estimate fits ``memory_fraction`` of the free memory."""
    config = config or PrefillConfig()
    if config.chunk_size > 0:
        return config.chunk_size
    if free_bytes is None:
        free_bytes = torch.cuda.mem_get_info()[0] if torch.cuda.is_available() else 8 << 30
    budget = int(free_bytes * config.memory_fraction)
    c = config.max_chunk
    while c > config.min_chunk and estimate_chunk_bytes(cfg, c, total_tokens) > budget:
        c //= 2
    return max(config.min_chunk, c)


def chunked_prefill(lm, input_ids: Sequence[int], kv=None, block_table: Optional[torch.Tensor] = None,
                    config: Optional[PrefillConfig] = None, progress_callback: Optional[Callable[[int, int], None]] = None,
                    start: int = 0):
    """Run one prompt through ``lm`` (``MMFP4ForCausalLM``) chunk by chunk.  Returns ``(logits fp32 [vocab] of the last
    token, stats, kv, block_table)``; ``kv`` / ``block_table`` are created when not given (``start`` tokens are taken as
    cached already)."""
    config = config or PrefillConfig()
    ids = list(input_ids.reshape(-1).tolist() if isinstance(input_ids, torch.Tensor) else input_ids)
    n = len(ids)
    if n - start <= 0:
        raise ValueError("nothing to prefill")
    model = lm.model
    dev = model.device
    if kv is None:
        bs = 16
        nb = (n + bs - 1) // bs + 1
        kv = lm.new_cache(nb, bs)
        block_table = torch.arange(nb, dtype=torch.int32).view(1, nb)
    elif block_table is None:
        raise ValueError("a cache needs its block table")
    if block_table.shape[1] * kv.block_size < n:
        raise ValueError(f"the block table covers {block_table.shape[1] * kv.block_size} positions, the prompt has {n}")
    chunk = pick_chunk_size(model.cfg, n, config)
    stats = PrefillStats(total_tokens=n - start, flash_attention_used=bool(config.use_flash_attention and dev.type == "cuda"
                                                                           and ops.native_available()))
    cuda = dev.type == "cuda"
    if cuda:
        torch.cuda.reset_peak_memory_stats(dev)
        torch.cuda.synchronize(dev)
    t_all = time.perf_counter()
    done, logits = start, None
    while done < n:
        step = min(chunk, n - done)
        t0 = time.perf_counter()
        if config.use_flash_attention:
            logits = _prefill(model, kv, [ids[: done + step]], block_table, start=[done], chunk_tokens=step, max_batch_tokens=step)
        else:
            with ops.force_reference():
                logits = _prefill(model, kv, [ids[: done + step]], block_table, start=[done], chunk_tokens=step, max_batch_tokens=step)
        if cuda:
            torch.cuda.synchronize(dev)
        stats.chunk_times_ms.append((time.perf_counter() - t0) * 1e3)
        done += step
        stats.num_chunks += 1
        if progress_callback is not None:
            progress_callback(done, n)
    stats.prefill_time_ms = (time.perf_counter() - t_all) * 1e3
    stats.tokens_per_second = stats.total_tokens / max(stats.prefill_time_ms, 1e-6) * 1e3
    if cuda:
        stats.peak_memory_mb = torch.cuda.max_memory_allocated(dev) / 2 ** 20
    return logits[0], stats, kv, block_table


def parallel_kv_write(kv, layer_rows: Sequence[Tuple[int, torch.Tensor, torch.Tensor]], slots: torch.Tensor) -> None:
    """Write already rotated key / value rows of several layers into the paged pools in one pass: ``layer_rows`` holds
    ``(layer, k [n, Hkv, D], v [n, Hkv, D])`` (``v`` None for an MLA latent pool), ``slots`` int64 ``[n]`` the cache rows.
    bf16 pools take an indexed copy per pool; quantized pools re-quantize the rows with their per-row scales."""
    slots = slots.to(torch.int64)
    for li, k, v in layer_rows:
        for pool, rows in ((kv.k[li], k), (kv.v[li] if getattr(kv, "v", None) else None, v)):
            if pool is None or rows is None:
                continue
            if isinstance(pool, ops.FP8KV):
                pool.store(slots, rows.reshape(rows.shape[0], *pool.shape[1:]))
            else:
                pool.view(pool.shape[0], -1).index_copy_(0, slots, rows.reshape(rows.shape[0], -1).to(pool.dtype))


def flash_prefill_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = True, scale: Optional[float] = None,
                            window: int = 0) -> torch.Tensor:
    """``q [B, Hq, T, D]``, ``k, v [B, Hkv, N, D]`` (the queries are the last ``T`` positions of the ``N`` keys) ->
    ``[B, Hq, T, D]``.  Every sequence of the batch becomes one entry of a varlen call, so long single sequences reach the
    tcgen05 kernel and everything else the mma.sync kernel (or the PyTorch restatement on CPU)."""
    B, Hq, T, D = q.shape
    N = k.shape[2]
    qf = q.permute(0, 2, 1, 3).reshape(B * T, Hq, D).contiguous()
    kf = k.permute(0, 2, 1, 3).reshape(B * N, k.shape[1], D).contiguous()
    vf = v.permute(0, 2, 1, 3).reshape(B * N, v.shape[1], v.shape[3]).contiguous()
    if B == 1:
        cu_q = torch.tensor([0, T], dtype=torch.int32, device=q.device)
        cu_k = torch.tensor([0, N], dtype=torch.int32, device=q.device)
        out = ops.prefill_attention(qf, kf, vf, cu_q, cu_k=cu_k, max_q=T, scale=scale, window=window, causal=causal)
        return out.view(1, T, Hq, -1).permute(0, 2, 1, 3)
    cu_q = torch.arange(0, (B + 1) * T, T, dtype=torch.int32, device=q.device)
    cu_k = torch.arange(0, (B + 1) * N, N, dtype=torch.int32, device=q.device)
    out = ops.prefill_attention(qf, kf, vf, cu_q, cu_k=cu_k, max_q=T, scale=scale, window=window, causal=causal)
    return out.view(B, T, Hq, -1).permute(0, 2, 1, 3)


@dataclass
class SpeculativePrefillConfig:
    enabled: bool = False
    num_speculative_tokens: int = 4
    confidence_threshold: float = 0.9


def speculative_prefill(lm, input_ids: Sequence[int], kv, block_table: torch.Tensor,
                        config: Optional[SpeculativePrefillConfig] = None, start: int = 0):
    """Prefill, then greedily extend the cache by up to ``num_speculative_tokens`` tokens while the model's top probability
    stays at or above ``confidence_threshold``.  Returns ``(logits after the last cached token, speculated token ids)``: a
    decode loop whose next tokens equal the speculated ones continues from ``len(prompt) + len(speculated)`` with those
    logits; on the first mismatch it resumes at that position (the rows behind it are simply overwritten)."""
    config = config or SpeculativePrefillConfig()
    ids = list(input_ids.reshape(-1).tolist() if isinstance(input_ids, torch.Tensor) else input_ids)
    logits = _prefill(lm.model, kv, [ids], block_table, start=[start])[0]
    spec: List[int] = []
    if not config.enabled:
        return logits, spec
    room = block_table.shape[1] * kv.block_size - len(ids)
    for _ in range(min(config.num_speculative_tokens, room)):
        p = torch.softmax(logits.float(), -1)
        conf, tok = p.max(-1)
        if float(conf) < config.confidence_threshold:
            break
        spec.append(int(tok))
        ids.append(int(tok))
        logits = _prefill(lm.model, kv, [ids], block_table, start=[len(ids) - 1])[0]
    return logits, spec
