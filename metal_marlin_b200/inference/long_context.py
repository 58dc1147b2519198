"""Long-context helpers: sliding-window + global-token masks, KV compression, streaming (sink) attention and
chunked memory-efficient attention.

Parity: reference ``metal_marlin/inference/long_context.py`` — ``LongContextConfig`` (``:40``), sliding window
with global tokens (``:90``), KV compression at ratio 4 above 8192 tokens (``:143``), streaming attention
(``:269``), chunked attention (``:379``) and ``LongContextModel`` (``:456``).  The reference carries
``use_sequence_parallel`` / ``sp_degree`` flags that nothing reads; here sequence parallelism over GPUs is the
ring exchange in ``parallel/cp.py`` and the flags select it.  The decode-time window is implemented in the
paged attention kernel (``window`` argument); these PyTorch forms serve prefill and are the oracle.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch
import torch.nn.functional as F


@dataclass
class LongContextConfig:
    max_context: int = 131072
    sliding_window: int = 4096
    global_tokens: int = 4              # attention sinks that every query sees
    compression_ratio: int = 4
    compression_threshold: int = 8192   # compress KV older than this many tokens
    chunk_size: int = 2048
    use_sequence_parallel: bool = False
    sp_degree: int = 1


def sliding_window_mask(q_len: int, kv_len: int, window: int, global_tokens: int = 0, device=None) -> torch.Tensor:
    """Boolean ``[q_len, kv_len]`` (True = attend): causal, within ``window`` of the query, or a global token.
    Queries are the last ``q_len`` positions of the ``kv_len`` keys."""
    qpos = torch.arange(kv_len - q_len, kv_len, device=device)[:, None]
    kpos = torch.arange(kv_len, device=device)[None, :]
    causal = kpos <= qpos
    near = (qpos - kpos) < window
    return causal & (near | (kpos < global_tokens))


def compress_kv(k: torch.Tensor, v: torch.Tensor, cfg: LongContextConfig) -> Tuple[torch.Tensor, torch.Tensor]:
    """Mean-pool the KV older than ``compression_threshold`` tokens in groups of ``compression_ratio`` along the
    sequence axis (``[B, H, S, D]``); the recent window and the global tokens stay exact."""
    S = k.shape[2]
    if S <= cfg.compression_threshold:
        return k, v
    g, r = cfg.global_tokens, cfg.compression_ratio
    old_end = S - cfg.compression_threshold
    old_end = g + ((old_end - g) // r) * r
    if old_end <= g:
        return k, v

    def pool(x):
        old = x[:, :, g:old_end]
        B, H, n, D = old.shape
        return torch.cat([x[:, :, :g], old.reshape(B, H, n // r, r, D).mean(3), x[:, :, old_end:]], 2)

    return pool(k), pool(v)


def chunked_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, chunk_size: int = 2048, causal: bool = True,
                      scale: Optional[float] = None, window: int = 0, global_tokens: int = 0) -> torch.Tensor:
    """Memory-efficient attention: queries in chunks, keys in chunks, online softmax in fp32.  ``[B, H, S, D]``
    (GQA: ``k``/``v`` may have fewer heads)."""
    B, H, Sq, D = q.shape
    Hk, Sk = k.shape[1], k.shape[2]
    if Hk != H:
        k, v = k.repeat_interleave(H // Hk, 1), v.repeat_interleave(H // Hk, 1)
    scale = scale if scale is not None else D ** -0.5
    out = torch.empty(B, H, Sq, v.shape[-1], dtype=q.dtype, device=q.device)
    off = Sk - Sq
    for q0 in range(0, Sq, chunk_size):
        q1 = min(Sq, q0 + chunk_size)
        qc = q[:, :, q0:q1].to(torch.float32) * scale
        m = torch.full((B, H, q1 - q0, 1), float("-inf"), device=q.device)
        l = torch.zeros(B, H, q1 - q0, 1, device=q.device)
        acc = torch.zeros(B, H, q1 - q0, v.shape[-1], device=q.device)
        k_hi = min(Sk, off + q1) if causal else Sk
        for k0 in range(0, k_hi, chunk_size):
            k1 = min(k_hi, k0 + chunk_size)
            s = qc @ k[:, :, k0:k1].to(torch.float32).transpose(-1, -2)
            qpos = torch.arange(off + q0, off + q1, device=q.device)[:, None]
            kpos = torch.arange(k0, k1, device=q.device)[None, :]
            ok = torch.ones(q1 - q0, k1 - k0, dtype=torch.bool, device=q.device)
            if causal:
                ok &= kpos <= qpos
            if window > 0:
                ok &= ((qpos - kpos) < window) | (kpos < global_tokens)
            s = s.masked_fill(~ok, float("-inf"))
            m_new = torch.maximum(m, s.amax(-1, keepdim=True))
            m_safe = torch.where(torch.isinf(m_new), torch.zeros_like(m_new), m_new)
            p = torch.exp(s - m_safe)
            corr = torch.exp(torch.where(torch.isinf(m), torch.full_like(m, float("-inf")), m - m_safe))
            l = l * corr + p.sum(-1, keepdim=True)
            acc = acc * corr + p @ v[:, :, k0:k1].to(torch.float32)
            m = m_new
        out[:, :, q0:q1] = (acc / l.clamp_min(1e-30)).to(q.dtype)
    return out


class StreamingAttention:
    """Attention-sink streaming: keeps ``global_tokens`` sinks + the last ``sliding_window`` tokens of K/V and
    attends over them only, so memory is bounded for an unbounded stream."""

    def __init__(self, cfg: LongContextConfig):
        self.cfg = cfg
        self.k: Optional[torch.Tensor] = None
        self.v: Optional[torch.Tensor] = None

    def append(self, k: torch.Tensor, v: torch.Tensor):
        self.k = k if self.k is None else torch.cat([self.k, k], 2)
        self.v = v if self.v is None else torch.cat([self.v, v], 2)
        g, w = self.cfg.global_tokens, self.cfg.sliding_window
        if self.k.shape[2] > g + w:
            self.k = torch.cat([self.k[:, :, :g], self.k[:, :, -w:]], 2)
            self.v = torch.cat([self.v[:, :, :g], self.v[:, :, -w:]], 2)

    def __call__(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
        self.append(k, v)
        return chunked_attention(q, self.k, self.v, self.cfg.chunk_size, causal=True)


class LongContextModel:
    """Drives a causal LM over a long prompt in ``chunk_size`` pieces (chunked prefill through the paged cache)
    and reports which strategy each range used."""

    def __init__(self, lm, cfg: Optional[LongContextConfig] = None):
        self.lm, self.cfg = lm, cfg or LongContextConfig()

    def prefill(self, token_ids, kv, block_tables):
        from ..models.mmfp4_causal_lm import prefill
        if len(token_ids) > self.cfg.max_context:
            raise ValueError(f"prompt of {len(token_ids)} tokens exceeds max_context {self.cfg.max_context}")
        return prefill(self.lm.model, kv, [list(token_ids)], block_tables, chunk_tokens=self.cfg.chunk_size)
