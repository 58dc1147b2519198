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


# ------------------------------------------------------------------------------------------ block-sparse mask object
class BlockSparseMask:
    """Which (query block, key block) pairs are computed, stored as bit sets: ``mask_bits [num_q_blocks, ceil(num_k_blocks / 64)]``
    int64 words (the bit pattern of unsigned 64-bit words: bit ``j % 64`` of word ``j // 64`` in row ``i`` says that query block ``i``
    attends to key block ``j``).  Factories for the usual patterns; ``dense()`` gives the boolean block matrix the attention
    entry points take.  Reference ``attention.py:40`` (``BlockSparseMask``: ``create_sliding_window`` / ``create_bigbird`` /
    ``create_longformer`` / ``from_dense_mask``)."""

    def __init__(self, mask_bits: torch.Tensor, block_q: int, block_k: int, num_q_blocks: int, num_k_blocks: int, seq_q: int, seq_k: int):
        self.mask_bits, self.block_q, self.block_k = mask_bits, block_q, block_k
        self.num_q_blocks, self.num_k_blocks, self.seq_q, self.seq_k = num_q_blocks, num_k_blocks, seq_q, seq_k

    @classmethod
    def from_block_matrix(cls, blocks: torch.Tensor, block_q: int, block_k: int, seq_q: int, seq_k: int, device=None) -> "BlockSparseMask":
        b = blocks.bool().cpu()
        nq, nk = b.shape
        words = (nk + 63) // 64
        pad = torch.zeros(nq, words * 64, dtype=torch.int64)
        pad[:, :nk] = b.long()
        shifts = torch.arange(64, dtype=torch.int64)
        lo = (pad.view(nq, words, 64)[..., :63] << shifts[:63]).sum(-1)
        top = pad.view(nq, words, 64)[..., 63]
        bits = lo | torch.where(top > 0, torch.tensor(-2 ** 63, dtype=torch.int64), torch.tensor(0, dtype=torch.int64))
        return cls(bits.to(device) if device is not None else bits, block_q, block_k, nq, nk, seq_q, seq_k)

    def dense(self) -> torch.Tensor:
        """bool ``[num_q_blocks, num_k_blocks]``."""
        w = self.mask_bits.cpu()
        shifts = torch.arange(64, dtype=torch.int64)
        bits = ((w.unsqueeze(-1) >> shifts) & 1).bool().reshape(self.num_q_blocks, -1)
        return bits[:, : self.num_k_blocks]

    def is_active(self, q_block: int, k_block: int) -> bool:
        return bool((int(self.mask_bits[q_block, k_block // 64]) >> (k_block % 64)) & 1)

    @property
    def density(self) -> float:
        return float(self.dense().float().mean())

    def element_mask(self, causal: bool = False) -> torch.Tensor:
        """bool ``[seq_q, seq_k]`` (queries are the last positions of the keys for the causal rule)."""
        m = self.dense().repeat_interleave(self.block_q, 0).repeat_interleave(self.block_k, 1)[: self.seq_q, : self.seq_k]
        if causal:
            qpos = torch.arange(self.seq_q).unsqueeze(1) + (self.seq_k - self.seq_q)
            m = m & (torch.arange(self.seq_k).unsqueeze(0) <= qpos)
        return m

    @staticmethod
    def _blocks(seq_len: int, block_size: int) -> int:
        return (seq_len + block_size - 1) // block_size

    @classmethod
    def create_sliding_window(cls, seq_len: int, window_size: int, block_size: int = 64, device=None) -> "BlockSparseMask":
        """Causal sliding window: query block ``i`` sees the key blocks that hold any position within ``window_size`` before its
        last query, up to itself."""
        n = cls._blocks(seq_len, block_size)
        qi = torch.arange(n)
        q_end = torch.clamp((qi + 1) * block_size, max=seq_len)
        first = torch.clamp(q_end - window_size, min=0) // block_size
        kj = torch.arange(n).unsqueeze(0)
        return cls.from_block_matrix((kj >= first.unsqueeze(1)) & (kj <= qi.unsqueeze(1)), block_size, block_size, seq_len, seq_len, device)

    @classmethod
    def create_bigbird(cls, seq_len: int, num_random_blocks: int = 3, num_global_blocks: int = 2, window_size: int = 256, block_size: int = 64,
                       device=None, seed: int = 42) -> "BlockSparseMask":
        """Local window (both directions) + the first ``num_global_blocks`` blocks seen by and seeing everything + ``num_random_blocks``
        further key blocks visible to every query (drawn once with ``seed``)."""
        n = cls._blocks(seq_len, block_size)
        w = max(1, window_size // block_size)
        idx = torch.arange(n)
        m = (idx.unsqueeze(0) - idx.unsqueeze(1)).abs() <= w // 2 if w > 1 else torch.eye(n, dtype=torch.bool)
        g = min(num_global_blocks, n)
        m[:, :g] = True
        m[:g, :] = True
        if num_random_blocks > 0 and n > g:
            gen = torch.Generator().manual_seed(seed)
            m[:, torch.randperm(n - g, generator=gen)[:num_random_blocks] + g] = True
        return cls.from_block_matrix(m, block_size, block_size, seq_len, seq_len, device)

    @classmethod
    def create_longformer(cls, seq_len: int, window_size: int = 512, global_token_indices: Sequence[int] = (0,), block_size: int = 64, device=None
                          ) -> "BlockSparseMask":
        """Symmetric local window + global tokens (their blocks attend everywhere and are attended from everywhere)."""
        n = cls._blocks(seq_len, block_size)
        idx = torch.arange(n)
        half = max(0, (window_size // 2 + block_size - 1) // block_size)
        m = (idx.unsqueeze(0) - idx.unsqueeze(1)).abs() <= half
        for t in global_token_indices:
            if 0 <= t < seq_len:
                m[t // block_size, :] = True
                m[:, t // block_size] = True
        return cls.from_block_matrix(m, block_size, block_size, seq_len, seq_len, device)

    @classmethod
    def from_dense_mask(cls, mask: torch.Tensor, block_q: int = 64, block_k: int = 64, device=None) -> "BlockSparseMask":
        """From an element mask ``[seq_q, seq_k]`` (bool: True = attend; float: finite = attend): a block is active when any of
        its elements is."""
        keep = mask.bool() if mask.dtype == torch.bool else torch.isfinite(mask) & (mask > -1e30)
        sq, sk = keep.shape
        nq, nk = (sq + block_q - 1) // block_q, (sk + block_k - 1) // block_k
        pad = torch.zeros(nq * block_q, nk * block_k, dtype=torch.bool)
        pad[:sq, :sk] = keep.cpu()
        return cls.from_block_matrix(pad.view(nq, block_q, nk, block_k).any(3).any(1), block_q, block_k, sq, sk, device)


def block_sparse_attention_metal(q, k, v, block_sparse_mask: BlockSparseMask, scale: Optional[float] = None, causal: bool = False):
    """``q [B, H, Sq, D]``, ``k / v [B, Hk, Sk, D]`` restricted to the active blocks of the mask (and to the causal triangle with
    ``causal``).  Square problems with one block size go to :func:`block_sparse_attention` (the prefill kernel skips empty key
    tiles on a GPU); others use the element mask.  Reference ``attention.py:900``."""
    m = block_sparse_mask
    if q.shape[2] != m.seq_q or k.shape[2] != m.seq_k:
        raise ValueError(f"sequence length mismatch: q={q.shape[2]}, k={k.shape[2]}, mask=({m.seq_q}, {m.seq_k})")
    if m.seq_q == m.seq_k and m.block_q == m.block_k and q.shape[1] == k.shape[1]:
        return block_sparse_attention(q, k, v, m.dense(), m.block_q, causal, scale)
    el = m.element_mask(causal).to(q.device)
    if k.shape[1] != q.shape[1]:
        k, v = k.repeat_interleave(q.shape[1] // k.shape[1], 1), v.repeat_interleave(q.shape[1] // v.shape[1], 1)
    return F.scaled_dot_product_attention(q, k, v, attn_mask=el, scale=scale)


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
