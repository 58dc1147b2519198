"""Decode-phase helpers: a persistent decode state (fixed buffers, the step captured in a CUDA graph), kernel selection by
problem size, and attention over quantized KV caches in the contiguous ``[batch, heads, seq, dim]`` layout.

Parity: reference ``metal_marlin/inference/decode.py`` (``DecodeConfig`` ``:72``, ``DecodePerfStats`` ``:161``, ``DecodeState``
``:193`` with its persistent buffers, ``select_decode_kernel`` ``:507``, ``quantized_kv_attention`` ``:697``,
``persistent_decode_step`` ``:913``).  The reference keeps per-layer output buffers alive between calls to avoid
allocations; here the whole step (all layers, sampling, cache bookkeeping) is one captured graph over fixed buffers
(``engine.session.DecodeSession``), which removes the allocations and the launch overhead together.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import torch

from .. import ops
from ..engine.session import DecodeSession, SamplingParams


@dataclass
class DecodeConfig:
    batch_size: int = 1
    max_context: int = 4096
    block_size: int = 16
    kv_cache_dtype: str = "bf16"          # bf16 | fp8 | int8 | fp4 | int4
    use_graph: Optional[bool] = None      # None: capture on CUDA devices
    max_new_tokens: int = 256


@dataclass
class DecodePerfStats:
    step_times_ms: List[float] = field(default_factory=list)
    weight_read_mb: float = 0.0
    kv_cache_read_mb: float = 0.0

    @property
    def total_time_ms(self) -> float:
        return float(sum(self.step_times_ms))

    @property
    def tokens_per_second(self) -> float:
        return 1e3 * len(self.step_times_ms) / self.total_time_ms if self.step_times_ms else 0.0

    @property
    def achieved_bandwidth_gbps(self) -> float:
        """Weight + cache bytes of the timed steps over their time."""
        if not self.step_times_ms:
            return 0.0
        return (self.weight_read_mb + self.kv_cache_read_mb) * len(self.step_times_ms) / 1e3 / (self.total_time_ms / 1e3)


class DecodeState:
    """Persistent decode state of ``lm`` (``MMFP4ForCausalLM``) for a fixed batch: the paged cache, the block tables, the
    token / position / slot buffers and the captured step.  ``prefill`` fills the cache and primes the first token;
    ``persistent_decode_step`` advances every sequence by one token without allocating."""

    def __init__(self, lm, config: Optional[DecodeConfig] = None):
        self.lm = lm
        self.config = config = config or DecodeConfig()
        B, bs = config.batch_size, config.block_size
        self.blocks_per_seq = (config.max_context + bs - 1) // bs
        self.kv = lm.new_cache(B * self.blocks_per_seq, bs, kv_dtype=config.kv_cache_dtype)
        self.block_tables = torch.arange(B * self.blocks_per_seq, dtype=torch.int32).view(B, self.blocks_per_seq)
        self.session = DecodeSession(lm.model, self.kv, B, self.blocks_per_seq, max_new_tokens=config.max_new_tokens,
                                     use_graph=config.use_graph, max_ctx=config.max_context)
        self.stats = DecodePerfStats()
        self.lengths = [0] * B
        cfg = lm.model.cfg
        # FP4 codes + one fp16 scale per 128 weights
        self.stats.weight_read_mb = cfg.param_count()["active"] * (0.5 + 2.0 / max(1, cfg.group_size)) / 2 ** 20

    def prefill(self, prompts: Sequence[Sequence[int]], sampling: Optional[Sequence[SamplingParams]] = None) -> torch.Tensor:
        """Write the prompts into the cache and return the first generated token of every sequence (greedy)."""
        from ..models.mmfp4_causal_lm import prefill
        assert len(prompts) == self.config.batch_size
        for p in prompts:
            if len(p) + self.config.max_new_tokens > self.config.max_context:
                raise ValueError("prompt + max_new_tokens exceeds max_context")
        logits = prefill(self.lm.model, self.kv, [list(p) for p in prompts], self.block_tables)
        first = logits.argmax(-1)
        self.lengths = [len(p) for p in prompts]
        if sampling is not None:
            self.session.set_sampling(sampling)
        self.session.set_state(first, self.lengths, self.block_tables)
        per_tok = sum(p.nbytes() // p.shape[0] if isinstance(p, ops.FP8KV) else p[0].numel() * p.element_size()
                      for pools in (self.kv.k, self.kv.v) for p in pools if p is not None)
        self.stats.kv_cache_read_mb = per_tok * sum(self.lengths) / 2 ** 20
        return first

    @property
    def tokens(self) -> torch.Tensor:
        """Current token of every sequence (device tensor, updated in place by every step)."""
        return self.session.ids


def persistent_decode_step(state: DecodeState, timed: bool = False) -> torch.Tensor:
    """One decode step for every sequence of ``state`` (graph replay on CUDA).  Returns the sampled ids (the session's own
    buffer: copy it to keep it).  ``timed`` synchronises and records the step time in ``state.stats``."""
    dev = state.session.device
    if timed:
        if dev.type == "cuda":
            torch.cuda.synchronize(dev)
        t0 = time.perf_counter()
    out = state.session.step()
    if timed:
        if dev.type == "cuda":
            torch.cuda.synchronize(dev)
        state.stats.step_times_ms.append((time.perf_counter() - t0) * 1e3)
    state.lengths = [n + 1 for n in state.lengths]
    return out


def select_decode_kernel(M: int, N: int, K: int) -> str:
    """Name of the kernel an FP4 projection ``[M, K] x [N, K]^T`` takes under the installed thresholds."""
    from ..autotune import get_optimal_config
    lim = get_optimal_config(M, N, K)["limit"]
    if M > lim and not ops.NO_TCGEN05:
        return "fp4_gemm_tcgen05"
    if M <= ops.GEMV_FUSED_PROLOGUE_MAX_M:
        return "fp4_gemv_fused_prologue"          # residual add + RMSNorm in the activation staging
    return "fp4_gemv_two_row_blocks" if 16 * (K + 32) * 2 + 8 * 4 * 640 <= 204 * 1024 else "fp4_gemv"


def quantize_kv_cache(x: torch.Tensor, quant_dtype: str = "fp8"):
    """``x [B, Hkv, S, D]`` -> ``(codes uint8 [B, Hkv, S, D or D / 2], scales fp32 [B, Hkv, S])`` in the engine's KV formats
    (one scale per cached row and head)."""
    B, H, S, D = x.shape
    pool = ops.FP8KV(B * S, (H, D), x.device, quant_dtype)
    pool.store(torch.arange(B * S, device=x.device), x.permute(0, 2, 1, 3).reshape(B * S, H, D))
    return (pool.data.view(B, S, H, -1).permute(0, 2, 1, 3).contiguous(), pool.scale.view(B, S, H).permute(0, 2, 1).contiguous())


def quantized_kv_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, k_scales: torch.Tensor,
                           v_scales: torch.Tensor, num_heads: int, num_kv_heads: int, seq_lens: Optional[torch.Tensor] = None,
                           quant_dtype: str = "fp8", scale: Optional[float] = None, window: int = 0) -> torch.Tensor:
    """Decode attention of ``q [B, Hq, 1, D]`` over quantized caches ``[B, Hkv, S, W]`` with scales ``[B, Hkv, S]`` (as
    ``quantize_kv_cache`` returns them).  The caches are viewed as paged pools of 16-row blocks and go to the paged decode
    kernel, which expands the codes in shared memory; ``seq_lens`` int32 ``[B]`` (default: all ``S``).  Returns ``[B, Hq, 1, D]``."""
    B, Hq, _, D = q.shape
    S = k_cache.shape[2]
    bs = 16
    S_pad = (S + bs - 1) // bs * bs
    dev = q.device

    def pool_of(codes, scales):
        p = ops.FP8KV(B * S_pad, (num_kv_heads, D), dev, quant_dtype)
        p.data.view(B, S_pad, num_kv_heads, -1)[:, :S].copy_(codes.permute(0, 2, 1, 3))
        p.scale.view(B, S_pad, num_kv_heads)[:, :S].copy_(scales.permute(0, 2, 1))
        return p
    kp, vp = pool_of(k_cache, k_scales), pool_of(v_cache, v_scales)
    bt = torch.arange(B * S_pad // bs, dtype=torch.int32, device=dev).view(B, S_pad // bs)
    cl = seq_lens.to(torch.int32).to(dev) if seq_lens is not None else torch.full((B,), S, dtype=torch.int32, device=dev)
    o = ops.paged_attention(q.reshape(B, Hq, D).contiguous(), kp, vp, bt, cl, Hq=num_heads, Hkv=num_kv_heads, dqk=D, dv=D,
                            block_size=bs, scale=scale if scale is not None else D ** -0.5, window=window)
    return o.reshape(B, Hq, 1, D)
