"""MoE routing analysis: expert usage histograms, load imbalance, gate entropy, co-activation.

Parity: reference ``metal_marlin/analysis/moe_routing.py`` (routing profiler behind ``metal-marlin analyze``),
``metal_marlin/moe/*`` load-balancing tracker and gate-entropy helpers, ``metal_marlin/capacity.py`` (capacity
factor / token dropping).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch


class ExpertUsageProfiler:
    def __init__(self, num_layers: int, num_experts: int):
        self.counts = torch.zeros(num_layers, num_experts, dtype=torch.int64)
        self.coact = torch.zeros(num_layers, num_experts, num_experts, dtype=torch.int64)
        self.entropy_sum = torch.zeros(num_layers, dtype=torch.float64)
        self.tokens = torch.zeros(num_layers, dtype=torch.int64)

    def record(self, layer: int, expert_ids: torch.Tensor, router_probs: Optional[torch.Tensor] = None):
        """``expert_ids [T, k]``; ``router_probs [T, E]`` (optional, for the gate entropy)."""
        ids = expert_ids.detach().cpu().long()
        E = self.counts.shape[1]
        self.counts[layer] += torch.bincount(ids.reshape(-1), minlength=E)
        onehot = torch.zeros(ids.shape[0], E, dtype=torch.int64).scatter_(1, ids, 1)
        self.coact[layer] += onehot.t() @ onehot
        self.tokens[layer] += ids.shape[0]
        if router_probs is not None:
            p = router_probs.detach().cpu().to(torch.float64).clamp_min(1e-30)
            self.entropy_sum[layer] += float(-(p * p.log()).sum(-1).sum())

    def summary(self) -> Dict:
        c = self.counts.to(torch.float64)
        tot = c.sum(1, keepdim=True).clamp_min(1)
        frac = c / tot
        E = c.shape[1]
        return {
            "load_imbalance": (frac.max(1).values * E).tolist(),                 # 1.0 = perfectly balanced
            "dead_experts": (c == 0).sum(1).tolist(),
            "usage_cv": (frac.std(1) / frac.mean(1).clamp_min(1e-30)).tolist(),
            "gate_entropy": (self.entropy_sum / self.tokens.clamp_min(1)).tolist(),
            "hottest": c.argmax(1).tolist(),
        }


def load_balancing_loss(router_probs: torch.Tensor, expert_ids: torch.Tensor, num_experts: int) -> torch.Tensor:
    """Switch-style auxiliary loss: ``E * sum_e f_e * P_e`` (fraction of tokens routed to e times mean gate prob)."""
    T = router_probs.shape[0]
    f = torch.zeros(num_experts, device=router_probs.device).scatter_add_(
        0, expert_ids.reshape(-1).long(), torch.ones(expert_ids.numel(), device=router_probs.device)) / max(T * expert_ids.shape[1], 1)
    return num_experts * (f * router_probs.mean(0)).sum()


def apply_capacity(expert_ids: torch.Tensor, weights: torch.Tensor, num_experts: int, capacity_factor: float = 1.25):
    """Token dropping: each expert keeps at most ``ceil(capacity_factor * T * k / E)`` assignments (earliest tokens
    win); dropped assignments get id -1 and weight 0.  Returns ``(ids, weights, dropped_count)``."""
    T, k = expert_ids.shape
    cap = int(-(-capacity_factor * T * k // num_experts))
    flat = expert_ids.reshape(-1).long()
    onehot = torch.nn.functional.one_hot(flat.clamp_min(0), num_experts)
    rank = (onehot.cumsum(0) * onehot).sum(1)                # 1-based arrival order within the expert
    keep = (rank <= cap) & (flat >= 0)
    ids = torch.where(keep, flat, torch.full_like(flat, -1)).view(T, k).to(expert_ids.dtype)
    w = torch.where(keep.view(T, k), weights, torch.zeros_like(weights))
    return ids, w, int((~keep).sum())
