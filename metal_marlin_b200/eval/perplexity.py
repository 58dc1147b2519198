"""Evaluation: sliding-window perplexity, KL divergence between two models' next-token distributions, top-1
agreement, and a quality report that compares a quantized model against its float source.

Parity: reference ``metal_marlin/eval/perplexity.py`` (WikiText-2 style strided windows: context ``max_length``,
stride ``stride``, only the tokens new to a window are scored), ``metal_marlin/eval/accuracy.py`` (KL / agreement)
and ``benchmarks/quality.py`` (the ``quality`` CLI).  ``logits_fn(ids) -> [T, V]`` is any callable; for the
engine's models use ``MMFP4ForCausalLM.forward_logits``.
"""
from __future__ import annotations

import math
from typing import Callable, Dict, List, Optional, Sequence

import torch
import torch.nn.functional as F

LogitsFn = Callable[[Sequence[int]], torch.Tensor]


def sliding_window_nll(logits_fn: LogitsFn, token_ids: Sequence[int], max_length: int = 2048, stride: int = 512) -> Dict[str, float]:
    """Mean negative log-likelihood over ``token_ids`` with overlapping windows."""
    ids = list(token_ids)
    n = len(ids)
    if n < 2:
        raise ValueError("need at least two tokens")
    total, count, prev_end = 0.0, 0, 0
    for begin in range(0, n, stride):
        end = min(begin + max_length, n)
        new = end - prev_end                       # tokens this window is responsible for
        if new <= 0:
            break
        window = ids[begin:end]
        logits = logits_fn(window).to(torch.float32)
        lp = torch.log_softmax(logits[:-1], -1)
        tgt = torch.tensor(window[1:], device=lp.device)
        nll = -lp.gather(1, tgt.view(-1, 1)).squeeze(1)
        take = min(new, nll.numel())
        total += float(nll[-take:].sum())
        count += take
        prev_end = end
        if end == n:
            break
    mean = total / max(count, 1)
    return {"nll": mean, "perplexity": math.exp(min(mean, 50.0)), "tokens": count}


def compute_perplexity(logits_fn: LogitsFn, token_ids: Sequence[int], max_length: int = 2048, stride: int = 512) -> float:
    return sliding_window_nll(logits_fn, token_ids, max_length, stride)["perplexity"]


def kl_divergence(ref_fn: LogitsFn, test_fn: LogitsFn, token_ids: Sequence[int], max_length: int = 2048) -> Dict[str, float]:
    """Mean / max KL(ref || test) per position and top-1 agreement."""
    kls: List[torch.Tensor] = []
    agree, total = 0, 0
    ids = list(token_ids)
    for b in range(0, len(ids), max_length):
        w = ids[b:b + max_length]
        if len(w) < 2:
            break
        lr = torch.log_softmax(ref_fn(w).to(torch.float32), -1)
        lt = torch.log_softmax(test_fn(w).to(torch.float32).to(lr.device), -1)
        kls.append((lr.exp() * (lr - lt)).sum(-1))
        agree += int((lr.argmax(-1) == lt.argmax(-1)).sum())
        total += lr.shape[0]
    kl = torch.cat(kls)
    return {"kl_mean": float(kl.mean()), "kl_max": float(kl.max()), "kl_p99": float(kl.quantile(0.99)),
            "top1_agreement": agree / max(total, 1), "positions": total}


def quality_report(ref_fn: LogitsFn, test_fn: LogitsFn, token_ids: Sequence[int], max_length: int = 2048, stride: int = 512) -> Dict:
    r = sliding_window_nll(ref_fn, token_ids, max_length, stride)
    t = sliding_window_nll(test_fn, token_ids, max_length, stride)
    kl = kl_divergence(ref_fn, test_fn, token_ids, max_length)
    return {"ref_perplexity": r["perplexity"], "test_perplexity": t["perplexity"],
            "perplexity_delta_pct": 100.0 * (t["perplexity"] / r["perplexity"] - 1.0), **kl}


def synthetic_corpus(vocab_size: int, n_tokens: int, seed: int = 0) -> List[int]:
    """Zipf-distributed token stream for offline smoke evaluation (no dataset download)."""
    g = torch.Generator().manual_seed(seed)
    ranks = torch.arange(1, vocab_size + 1, dtype=torch.float64)
    p = (1.0 / ranks) / (1.0 / ranks).sum()
    return torch.multinomial(p, n_tokens, replacement=True, generator=g).tolist()
