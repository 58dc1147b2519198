"""Calibration data and Hessian collection.

Parity: reference ``metal_marlin/calibration/*`` (calibration datasets ``bartowski-v3`` / ``wikitext2`` / ``c4``,
``HessianCollector`` accumulating ``X^T X`` per linear layer, per-expert Hessians for MoE).  This environment has
no network, so named datasets resolve to local text files when present (``$METAL_MARLIN_CALIBRATION_DIR``) and
otherwise to a deterministic synthetic token stream of the same shape.
"""
from __future__ import annotations

import os
from typing import Dict, Iterable, List, Optional, Sequence

import torch

KNOWN_DATASETS = ("bartowski-v3", "wikitext2", "c4", "synthetic")


def load_calibration_tokens(name: str, tokenizer=None, vocab_size: int = 32000, num_samples: int = 32, seq_len: int = 512,
                            seed: int = 0) -> List[List[int]]:
    """``num_samples`` token sequences of ``seq_len``."""
    path = None
    if os.path.isfile(name):
        path = name
    else:
        d = os.environ.get("METAL_MARLIN_CALIBRATION_DIR")
        if d and os.path.isfile(os.path.join(d, f"{name}.txt")):
            path = os.path.join(d, f"{name}.txt")
    if path is not None and tokenizer is not None:
        ids = tokenizer.encode(open(path, encoding="utf-8", errors="ignore").read())
        if len(ids) >= seq_len:
            n = min(num_samples, len(ids) // seq_len)
            return [ids[i * seq_len:(i + 1) * seq_len] for i in range(n)]
    if name not in KNOWN_DATASETS and path is None:
        raise ValueError(f"unknown calibration set {name!r} (known: {KNOWN_DATASETS}, or a text file path)")
    from ..eval.perplexity import synthetic_corpus
    stream = synthetic_corpus(vocab_size, num_samples * seq_len, seed)
    return [stream[i * seq_len:(i + 1) * seq_len] for i in range(num_samples)]


class HessianCollector:
    """Accumulates ``H = sum_t x_t x_t^T`` (fp32, on the activations' device) and the token count per named layer;
    ``add(name, x)`` takes ``x [..., in]``.  ``add_expert`` keeps one Hessian per expert from routed tokens."""

    def __init__(self):
        self.H: Dict[str, torch.Tensor] = {}
        self.n: Dict[str, int] = {}

    def add(self, name: str, x: torch.Tensor):
        X = x.reshape(-1, x.shape[-1]).to(torch.float32)
        if name not in self.H:
            self.H[name] = torch.zeros(X.shape[1], X.shape[1], device=X.device)
            self.n[name] = 0
        self.H[name].addmm_(X.t(), X)
        self.n[name] += X.shape[0]

    def add_expert(self, name: str, x: torch.Tensor, expert_ids: torch.Tensor, num_experts: int):
        X = x.reshape(-1, x.shape[-1])
        ids = expert_ids.reshape(X.shape[0], -1)
        for e in ids.unique().tolist():
            if e < 0:
                continue
            rows = (ids == e).any(1)
            self.add(f"{name}.experts.{e}", X[rows])

    def get(self, name: str, normalize: bool = True) -> Optional[torch.Tensor]:
        if name not in self.H:
            return None
        return self.H[name] / max(self.n[name], 1) if normalize else self.H[name]

    def names(self) -> List[str]:
        return sorted(self.H)

    def save(self, path: str):
        torch.save({"H": {k: v.cpu() for k, v in self.H.items()}, "n": self.n}, path)

    @classmethod
    def load(cls, path: str) -> "HessianCollector":
        d = torch.load(path, map_location="cpu")
        c = cls()
        c.H, c.n = d["H"], d["n"]
        return c
