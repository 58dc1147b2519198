"""Expert load tracking: exponential moving average of every expert's share of the routed tokens, hot / cold / dead expert
lists, the auxiliary balancing loss (Switch form, optionally with the router z-loss) and the gate entropy.

Parity: reference ``metal_marlin/trellis/load_balancing.py``: ``LoadBalancingConfig`` ``:42``, ``ExpertLoadTracker`` ``:69``
(``update`` ``:110``, ``compute_loss`` ``:150``, ``get_hot_experts`` ``:218``, ``get_cold_experts`` ``:225``, ``get_dead_experts``
``:233``), ``compute_load_balance_loss_inline`` ``:241``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch


@dataclass
class LoadBalancingConfig:
    num_experts: int = 64
    top_k: int = 4
    ema_decay: float = 0.99
    aux_loss_weight: float = 0.01
    z_loss_weight: float = 0.0
    dead_after_updates: int = 100        # an expert with no token for this many updates counts as dead


def load_balance_loss(router_probs: torch.Tensor, expert_ids: torch.Tensor, num_experts: int) -> torch.Tensor:
    """``E * sum_e f_e * P_e``: ``f_e`` the fraction of assignments that went to expert e, ``P_e`` its mean gate probability;
    1.0 when routing is uniform."""
    flat = expert_ids.reshape(-1).long()
    ok = flat >= 0
    f = torch.zeros(num_experts, device=router_probs.device, dtype=router_probs.dtype)
    f.scatter_add_(0, flat[ok], torch.ones(int(ok.sum()), device=router_probs.device, dtype=router_probs.dtype))
    f = f / f.sum().clamp_min(1)
    return num_experts * (f * router_probs.mean(0)).sum()


def gate_entropy(router_probs: torch.Tensor, normalized: bool = True) -> torch.Tensor:
    """Mean entropy of the routing distribution per token (``normalized``: divided by ``log E``, so 1 = uniform, 0 = one-hot)."""
    p = router_probs.to(torch.float64).clamp_min(1e-30)
    h = -(p * p.log()).sum(-1).mean()
    return (h / torch.log(torch.tensor(float(p.shape[-1]), dtype=torch.float64))).to(torch.float32) if normalized else h.to(torch.float32)


class ExpertLoadTracker:
    def __init__(self, config: Optional[LoadBalancingConfig] = None, **kw):
        self.cfg = config or LoadBalancingConfig(**kw)
        self.reset()

    def reset(self) -> None:
        E = self.cfg.num_experts
        self.ema = torch.full((E,), 1.0 / E, dtype=torch.float64)
        self.counts = torch.zeros(E, dtype=torch.int64)
        self.idle = torch.zeros(E, dtype=torch.int64)
        self.updates = 0
        self.entropy_ema: Optional[float] = None

    def update(self, expert_ids: torch.Tensor, router_probs: Optional[torch.Tensor] = None) -> None:
        E, d = self.cfg.num_experts, self.cfg.ema_decay
        flat = expert_ids.detach().reshape(-1).long().cpu()
        c = torch.bincount(flat[flat >= 0], minlength=E)
        self.counts += c
        share = c.to(torch.float64) / max(1, int(c.sum()))
        self.ema = d * self.ema + (1 - d) * share
        self.idle = torch.where(c > 0, torch.zeros_like(self.idle), self.idle + 1)
        self.updates += 1
        if router_probs is not None:
            h = float(gate_entropy(router_probs.detach().cpu()))
            self.entropy_ema = h if self.entropy_ema is None else d * self.entropy_ema + (1 - d) * h

    def compute_loss(self, router_probs: torch.Tensor, expert_ids: torch.Tensor, router_logits: Optional[torch.Tensor] = None) -> torch.Tensor:
        loss = self.cfg.aux_loss_weight * load_balance_loss(router_probs, expert_ids, self.cfg.num_experts)
        if self.cfg.z_loss_weight and router_logits is not None:
            loss = loss + self.cfg.z_loss_weight * torch.logsumexp(router_logits.float(), -1).pow(2).mean()
        return loss

    def get_expert_loads(self) -> torch.Tensor:
        """EMA load of every expert relative to the uniform share (1.0 = its fair share)."""
        return (self.ema * self.cfg.num_experts).to(torch.float32)

    def get_hot_experts(self, threshold: float = 1.5) -> List[int]:
        return (self.get_expert_loads() > threshold).nonzero().reshape(-1).tolist()

    def get_cold_experts(self, threshold: float = 0.5) -> List[int]:
        return (self.get_expert_loads() < threshold).nonzero().reshape(-1).tolist()

    def get_dead_experts(self) -> List[int]:
        return (self.idle >= self.cfg.dead_after_updates).nonzero().reshape(-1).tolist()

    def imbalance(self) -> float:
        """Largest EMA load over the fair share (1.0 = perfectly balanced): what an expert-parallel step waits for."""
        return float(self.get_expert_loads().max())
