"""Verification of drafted tokens: exact speculative (rejection) sampling, greedy matching, and
tree verification for EAGLE-style drafts.

Parity: reference ``metal_marlin/speculative/verify.py:98`` (``verify_speculative``: accept while
``r < p/q``, on the first rejection resample from ``norm(max(p - q, 0))``, bonus token when all are
accepted), ``:188`` (``verify_eagle_tree``) and the vectorised ``verify_kernel``
(``metal_marlin/layers/mmfp4_mtp_head.py:479``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch


@dataclass
class VerifyResult:
    num_accepted: int          # drafted tokens kept
    next_token: int            # token appended after the accepted prefix (resampled or bonus)
    accepted_mask: List[bool]


def verify_greedy(target_logits: torch.Tensor, draft_tokens: Sequence[int]) -> VerifyResult:
    """``target_logits [K+1, V]``: row i is the target's distribution for the position of draft i."""
    tgt = target_logits.argmax(-1).tolist()
    n = 0
    for d, t in zip(draft_tokens, tgt):
        if d != t:
            break
        n += 1
    return VerifyResult(n, int(tgt[n]), [i < n for i in range(len(draft_tokens))])


def verify_speculative(target_probs: torch.Tensor, draft_probs: Optional[torch.Tensor], draft_tokens: Sequence[int],
                       generator: Optional[torch.Generator] = None) -> VerifyResult:
    """Exact speculative sampling.  ``target_probs [K+1, V]``; ``draft_probs [K, V]`` or None for a
    deterministic draft (one-hot ``q``).  The output token sequence is distributed exactly as if it
    had been sampled from the target alone."""
    K = len(draft_tokens)
    u = torch.rand(K + 1, generator=generator, device="cpu")
    for i, d in enumerate(draft_tokens):
        p = float(target_probs[i, d])
        q = 1.0 if draft_probs is None else float(draft_probs[i, d])
        if q > 0 and float(u[i]) < min(1.0, p / q):
            continue
        resid = target_probs[i].clone().float()
        if draft_probs is None:
            resid[d] = 0.0
        else:
            resid = (resid - draft_probs[i].float()).clamp_min_(0.0)
        z = float(resid.sum())
        if z <= 0:
            resid = target_probs[i].float()
            z = float(resid.sum())
        nxt = int(torch.multinomial((resid / z).cpu(), 1, generator=generator))
        return VerifyResult(i, nxt, [j < i for j in range(K)])
    bonus = int(torch.multinomial(target_probs[K].float().cpu(), 1, generator=generator))
    return VerifyResult(K, bonus, [True] * K)


def verify_batch_greedy(target_logits: torch.Tensor, draft_tokens: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Vectorised greedy verification.  ``target_logits [B, K+1, V]``, ``draft_tokens [B, K]`` ->
    (num_accepted [B], next_token [B]) without a host sync."""
    tgt = target_logits.argmax(-1)                                    # [B, K+1]
    ok = (tgt[:, :-1] == draft_tokens).to(torch.int64)
    n_acc = ok.cumprod(dim=1).sum(dim=1)
    return n_acc, tgt.gather(1, n_acc.unsqueeze(1)).squeeze(1)


def tree_attention_mask(parents: Sequence[int], device=None) -> torch.Tensor:
    """Boolean ``[N, N]`` mask: node i may attend to node j iff j is i or an ancestor of i.
    ``parents[i]`` is the parent index (``-1`` for children of the root/context).
    Parity: reference ``metal_marlin/tree_attention.py:126-507``."""
    n = len(parents)
    m = torch.zeros(n, n, dtype=torch.bool, device=device)
    for i in range(n):
        j = i
        while j >= 0:
            m[i, j] = True
            j = parents[j]
    return m


def verify_tree_greedy(target_logits_root: torch.Tensor, target_logits_nodes: torch.Tensor, tokens: Sequence[int],
                       parents: Sequence[int]) -> Tuple[List[int], int]:
    """Walk the draft tree following the target's greedy choices.  ``target_logits_root [V]`` is the
    distribution after the context, ``target_logits_nodes [N, V]`` the distribution after each tree node.
    Returns (indices of accepted nodes root->leaf, next token)."""
    children = {}
    for i, p in enumerate(parents):
        children.setdefault(p, []).append(i)
    path, cur, logits = [], -1, target_logits_root
    while True:
        want = int(logits.argmax())
        nxt = next((c for c in children.get(cur, []) if tokens[c] == want), None)
        if nxt is None:
            return path, want
        path.append(nxt)
        cur, logits = nxt, target_logits_nodes[nxt]
