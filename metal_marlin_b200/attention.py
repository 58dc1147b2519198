"""Attention variants built on the op layer: block-sparse masks (sliding / BigBird / Longformer), sliding-window
attention, tree attention for speculative decoding, and differential attention.

Parity: reference ``metal_marlin/attention.py`` (block-sparse mask builders), ``sliding_window_attention.py``,
``tree_attention.py:126-507`` (tree mask from parent pointers, tree-verify attention) and
``architectures/diff_transformer.py`` (two softmax maps subtracted with a learned lambda, per-head RMS norm).
These are PyTorch forms (prefill-side / oracle); decode runs in ``csrc/attention_decode.cu``.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence

import torch
import torch.nn.functional as F


# ------------------------------------------------------------------------------------------ block-sparse masks
def block_mask_sliding(n_blocks: int, window_blocks: int, causal: bool = True) -> torch.Tensor:
    i = torch.arange(n_blocks)[:, None]
    j = torch.arange(n_blocks)[None, :]
    m = (i - j).abs() < window_blocks
    return m & (j <= i) if causal else m


def block_mask_bigbird(n_blocks: int, window_blocks: int = 3, global_blocks: int = 1, random_blocks: int = 1, seed: int = 0,
                       causal: bool = True) -> torch.Tensor:
    m = block_mask_sliding(n_blocks, window_blocks, causal=False)
    m[:, :global_blocks] = True
    m[:global_blocks, :] = True
    g = torch.Generator().manual_seed(seed)
    for i in range(n_blocks):
        if random_blocks:
            m[i, torch.randint(0, n_blocks, (random_blocks,), generator=g)] = True
    if causal:
        m &= torch.tril(torch.ones(n_blocks, n_blocks, dtype=torch.bool))
    return m


def block_mask_longformer(n_blocks: int, window_blocks: int, global_block_ids: Sequence[int] = (0,), causal: bool = True) -> torch.Tensor:
    m = block_mask_sliding(n_blocks, window_blocks, causal=False)
    for gidx in global_block_ids:
        m[:, gidx] = True
        m[gidx, :] = True
    if causal:
        m &= torch.tril(torch.ones(n_blocks, n_blocks, dtype=torch.bool))
    return m


def expand_block_mask(block_mask: torch.Tensor, block: int, seq_len: int, causal: bool = True) -> torch.Tensor:
    m = block_mask.repeat_interleave(block, 0).repeat_interleave(block, 1)[:seq_len, :seq_len]
    if causal:
        m = m & torch.tril(torch.ones(seq_len, seq_len, dtype=torch.bool, device=m.device))
    return m


def _kernel_ok(q, k, v) -> bool:
    """Whether the varlen prefill kernel serves these ``[B, H, S, D]`` operands (bf16 on a GPU, supported head size)."""
    from . import ops
    return (q.is_cuda and ops.native_available() and q.dtype == torch.bfloat16 and k.dtype == torch.bfloat16
            and q.shape[-1] in ops.PREFILL_ATTN_DIMS and k.shape[-1] == q.shape[-1] == v.shape[-1] and q.shape[1] % k.shape[1] == 0)


def _kernel_call(q, k, v, scale, **mask_kw):
    """``[B, H, S, D]`` operands through ``ops.prefill_attention`` (token-major varlen layout, equal lengths)."""
    from . import ops
    B, H, S, D = q.shape
    N = k.shape[2]
    tm = lambda x: x.transpose(1, 2).reshape(B * x.shape[2], x.shape[1], D)
    cu_q = torch.arange(B + 1, dtype=torch.int32, device=q.device) * S
    cu_k = torch.arange(B + 1, dtype=torch.int32, device=q.device) * N
    o = ops.prefill_attention(tm(q), tm(k), tm(v), cu_q, cu_k=cu_k, max_q=S, scale=scale, **mask_kw)
    return o.view(B, S, H, D).transpose(1, 2)


def block_sparse_attention(q, k, v, block_mask: torch.Tensor, block: int = 64, causal: bool = True, scale=None):
    """``[B, H, S, D]`` attention restricted to the allowed blocks.  On the GPU the prefill kernel skips key tiles whose
    128-query x 64-key block is empty; masks finer than that ride along as an element mask."""
    S = q.shape[2]
    if _kernel_ok(q, k, v) and k.shape[2] == S:
        bm = block_mask.to(q.device).bool()
        el = bm.repeat_interleave(block, 0).repeat_interleave(block, 1)[:S, :S]          # element level, before causal
        nq, nk = (S + 127) // 128, (S + 63) // 64
        pad = torch.zeros(nq * 128, nk * 64, dtype=torch.bool, device=q.device)
        pad[:S, :S] = el
        coarse = pad.view(nq, 128, nk, 64).any(3).any(1).to(torch.uint8).unsqueeze(0).contiguous()
        exact = block % 128 == 0
        tree = None if exact else el.to(torch.uint8).repeat(q.shape[0], 1).contiguous()
        return _kernel_call(q, k, v, scale, causal=causal, block_mask=coarse, tree_mask=tree)
    m = expand_block_mask(block_mask.to(q.device), block, S, causal)
    return F.scaled_dot_product_attention(q, k, v, attn_mask=m, scale=scale)


def sliding_window_attention(q, k, v, window: int, global_tokens: int = 0, scale=None):
    from .inference.long_context import sliding_window_mask
    if _kernel_ok(q, k, v):
        return _kernel_call(q, k, v, scale, causal=True, window=window, sinks=global_tokens)
    m = sliding_window_mask(q.shape[2], k.shape[2], window, global_tokens, q.device)
    if k.shape[1] != q.shape[1]:
        k, v = k.repeat_interleave(q.shape[1] // k.shape[1], 1), v.repeat_interleave(q.shape[1] // v.shape[1], 1)
    return F.scaled_dot_product_attention(q, k, v, attn_mask=m, scale=scale)


# ------------------------------------------------------------------------------------------ tree attention
def tree_mask_from_parents(parents: Sequence[int]) -> torch.Tensor:
    """``parents[i]`` is the index of node i's parent (-1 = child of the last committed token).  Node i may attend
    to itself and its ancestors: boolean ``[N, N]``."""
    n = len(parents)
    m = torch.zeros(n, n, dtype=torch.bool)
    for i in range(n):
        j = i
        while j >= 0:
            m[i, j] = True
            j = parents[j]
    return m


def tree_attention(q, k_ctx, v_ctx, k_tree, v_tree, parents: Sequence[int], scale=None):
    """Queries are the N tree nodes ``[B, H, N, D]``; keys are the committed context (fully visible) followed by
    the tree nodes (ancestor-visible)."""
    N, C = q.shape[2], k_ctx.shape[2]
    k = torch.cat([k_ctx, k_tree], 2)
    v = torch.cat([v_ctx, v_tree], 2)
    if _kernel_ok(q, k, v):
        tm = tree_mask_from_parents(parents).to(device=q.device, dtype=torch.uint8).repeat(q.shape[0], 1).contiguous()
        return _kernel_call(q, k, v, scale, causal=False, tree_mask=tm)
    mask = torch.cat([torch.ones(N, C, dtype=torch.bool), tree_mask_from_parents(parents)], 1).to(q.device)
    return F.scaled_dot_product_attention(q, k, v, attn_mask=mask, scale=scale)


# ------------------------------------------------------------------------------------------ differential attention
def lambda_init_for_layer(layer_idx: int) -> float:
    return 0.8 - 0.6 * math.exp(-0.3 * layer_idx)


def differential_attention(q1, k1, q2, k2, v, lam: float, lambda_init: float, subln_weight: Optional[torch.Tensor] = None,
                           causal: bool = True, eps: float = 1e-5):
    """softmax(q1 k1^T) - lam * softmax(q2 k2^T), times v; per-head RMS norm; scaled by (1 - lambda_init)."""
    a1 = F.scaled_dot_product_attention(q1, k1, v, is_causal=causal)
    a2 = F.scaled_dot_product_attention(q2, k2, v, is_causal=causal)
    o = (a1 - lam * a2).to(torch.float32)
    o = o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + eps)
    if subln_weight is not None:
        o = o * subln_weight.to(torch.float32)
    return (o * (1.0 - lambda_init)).to(v.dtype)
