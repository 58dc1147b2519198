"""Speculative decoding: draft models (n-gram, small model, MTP heads, EAGLE), verification (greedy, rejection sampling,
token trees), acceptance tracking with adaptive depth, and the engines that drive them.

The names of the reference's ``metal_marlin.speculative`` package are available here (parity: its ``__init__`` exports
``SpeculativeConfig``, ``SpeculativeEngine``, ``DraftOutput`` / ``TreeDraftOutput``, ``VerifyResult`` / ``AcceptanceResult``,
``EagleHead`` + ``verify_eagle_tree``, ``MMFP4DraftModel``, acceptance statistics and reports,
``estimate_optimal_speculation_length``)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch

from .adaptive import AdaptiveSpeculationController, TokenAcceptanceTracker
from .draft import DraftModel, DraftOutput, EagleDraft, MTPDraft, MTPHead, NGramDraft, SmallModelDraft
from .engine import GenerationStats, SpeculativeEngine, make_draft
from .verify import (VerifyResult, tree_attention_mask, verify_batch_greedy, verify_greedy, verify_speculative,
                     verify_tree_greedy)

AcceptanceResult = VerifyResult
TreeDraftOutput = DraftOutput              # a draft with ``parents`` set is a tree
EagleHead = EagleDraft
MMFP4DraftModel = SmallModelDraft
AcceptanceStats = TokenAcceptanceTracker
StepResult = VerifyResult


@dataclass
class SpeculativeConfig:
    """Settings of a speculative engine: draft kind (``ngram`` | ``small`` | ``mtp`` | ``eagle``), tokens per step, adaptive
    depth and its bounds."""
    draft: str = "ngram"
    num_speculative_tokens: int = 4
    adaptive: bool = True
    min_depth: int = 1
    max_depth: int = 8
    draft_kwargs: Dict = field(default_factory=dict)

    def build(self, target_lm) -> SpeculativeEngine:
        return SpeculativeEngine(target_lm, make_draft(self.draft, target_lm, **self.draft_kwargs),
                                 num_speculative_tokens=self.num_speculative_tokens, adaptive=self.adaptive)


class MMFP4DraftModelWithTarget(SmallModelDraft):
    """A small-model draft that keeps a handle on its target (the reference pairs them to share embeddings / tokenizer)."""

    def __init__(self, draft_lm, target_lm=None, **kw):
        super().__init__(draft_lm, **kw)
        self.target = target_lm


@dataclass
class EagleTreeVerifyResult:
    accepted_path: List[int]          # node indices of the accepted root-to-leaf prefix
    tokens: List[int]                 # their tokens plus the token after them
    num_accepted: int


def verify_eagle_tree(target_logits_root: torch.Tensor, target_logits_nodes: torch.Tensor, tokens: Sequence[int],
                      parents: Sequence[int]) -> EagleTreeVerifyResult:
    """Greedy verification of a token tree: the longest path whose every token is the target's arg-max at its parent."""
    path, nxt = verify_tree_greedy(target_logits_root, target_logits_nodes, tokens, parents)
    return EagleTreeVerifyResult(list(path), [int(tokens[i]) for i in path] + [int(nxt)], len(path))


def compute_acceptance_probabilities(target_probs: torch.Tensor, draft_probs: torch.Tensor, draft_tokens: Sequence[int]) -> torch.Tensor:
    """``min(1, p_target / p_draft)`` of every drafted token (``[K]``)."""
    idx = torch.as_tensor(list(draft_tokens), dtype=torch.long, device=target_probs.device)
    k = idx.numel()
    p = target_probs[:k].gather(1, idx.view(-1, 1)).squeeze(1).float()
    q = draft_probs[:k].gather(1, idx.view(-1, 1)).squeeze(1).float().clamp_min(1e-30)
    return (p / q).clamp(max=1.0)


def estimate_optimal_speculation_length(acceptance_rate: float, draft_cost: float = 0.1, max_length: int = 16) -> int:
    """Draft length that maximises expected tokens per unit time when every drafted token is accepted independently with
    ``acceptance_rate`` and costs ``draft_cost`` of a target forward: ``E[tokens](k) = (1 - a^(k+1)) / (1 - a)`` over a step
    cost of ``1 + k * draft_cost``."""
    a = min(max(acceptance_rate, 0.0), 0.999999)
    best, best_v = 1, 0.0
    for k in range(1, max_length + 1):
        v = ((1 - a ** (k + 1)) / (1 - a)) / (1.0 + k * draft_cost)
        if v > best_v + 1e-12:
            best, best_v = k, v
    return best


def create_acceptance_report(tracker: TokenAcceptanceTracker) -> Dict:
    """Summary of an acceptance tracker: overall and recent rates, rate per draft position, expected tokens per step and
    the draft length :func:`estimate_optimal_speculation_length` suggests for the recent rate."""
    return {"proposed": tracker.total_proposed, "accepted": tracker.total_accepted, "acceptance_rate": tracker.acceptance_rate,
            "recent_rate": tracker.recent_rate, "position_rates": tracker.position_rates(),
            "expected_tokens_per_step": tracker.expected_tokens_per_step(),
            "suggested_length": estimate_optimal_speculation_length(tracker.recent_rate)}


__all__ = ["AcceptanceResult", "AcceptanceStats", "AdaptiveSpeculationController", "DraftModel", "DraftOutput", "EagleDraft", "EagleHead",
           "EagleTreeVerifyResult", "GenerationStats", "MMFP4DraftModel", "MMFP4DraftModelWithTarget", "MTPDraft", "MTPHead",
           "NGramDraft", "SmallModelDraft", "SpeculativeConfig", "SpeculativeEngine", "StepResult", "TokenAcceptanceTracker",
           "TreeDraftOutput", "VerifyResult", "compute_acceptance_probabilities", "create_acceptance_report",
           "estimate_optimal_speculation_length", "make_draft", "tree_attention_mask", "verify_batch_greedy", "verify_eagle_tree",
           "verify_greedy", "verify_speculative", "verify_tree_greedy"]
