"""Context (sequence) parallelism for long prompts: ring attention.

Every rank holds a contiguous slice of the sequence (queries, keys, values).  K/V slices travel around the ring;
each rank accumulates its queries' attention over the slices it has seen with an online softmax, skipping slices
that lie entirely in its causal future.  This is what the reference's ``use_sequence_parallel`` / ``sp_degree`` flags
(``metal_marlin/inference/long_context.py:40``) name but never implement.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist


def _merge(m, l, acc, s, v):
    """Online-softmax update of (running max, running sum, accumulator) with scores ``s [.., q, k]`` and values."""
    m_new = torch.maximum(m, s.amax(-1, keepdim=True))
    m_safe = torch.where(torch.isinf(m_new), torch.zeros_like(m_new), m_new)
    p = torch.exp(s - m_safe)
    corr = torch.exp(torch.where(torch.isinf(m), torch.full_like(m, float("-inf")), m - m_safe))
    return m_new, l * corr + p.sum(-1, keepdim=True), acc * corr + p @ v


def ring_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, group=None, causal: bool = True, scale: Optional[float] = None):
    """``q, k, v [B, H, S_local, D]`` - rank r owns positions ``[r * S_local, (r + 1) * S_local)``.  Returns this rank's
    attention output ``[B, H, S_local, Dv]``."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    B, H, S, D = q.shape
    if k.shape[1] != H:
        k, v = k.repeat_interleave(H // k.shape[1], 1), v.repeat_interleave(H // v.shape[1], 1)
    scale = scale if scale is not None else D ** -0.5
    qf = q.to(torch.float32) * scale
    m = torch.full((B, H, S, 1), float("-inf"), device=q.device)
    l = torch.zeros(B, H, S, 1, device=q.device)
    acc = torch.zeros(B, H, S, v.shape[-1], device=q.device)
    kv = torch.stack([k, v]).contiguous() if k.shape == v.shape else None
    cur_k, cur_v = k.contiguous(), v.contiguous()
    qpos = rank * S + torch.arange(S, device=q.device)[:, None]
    for step in range(world):
        src = (rank - step) % world                       # owner of the slice held right now
        if not (causal and src > rank):
            s = qf @ cur_k.to(torch.float32).transpose(-1, -2)
            if causal and src == rank:
                kpos = src * S + torch.arange(S, device=q.device)[None, :]
                s = s.masked_fill(kpos > qpos, float("-inf"))
            m, l, acc = _merge(m, l, acc, s, cur_v.to(torch.float32))
        if step + 1 < world:
            nxt_k, nxt_v = torch.empty_like(cur_k), torch.empty_like(cur_v)
            send_to, recv_from = (rank + 1) % world, (rank - 1) % world
            ops_ = [dist.P2POp(dist.isend, cur_k, send_to, group), dist.P2POp(dist.irecv, nxt_k, recv_from, group),
                    dist.P2POp(dist.isend, cur_v, send_to, group), dist.P2POp(dist.irecv, nxt_v, recv_from, group)]
            for w in dist.batch_isend_irecv(ops_):
                w.wait()
            cur_k, cur_v = nxt_k, nxt_v
    return (acc / l.clamp_min(1e-30)).to(q.dtype)
