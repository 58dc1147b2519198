"""Evaluation: sliding-window perplexity, KL divergence / agreement between two models, quality report, MoE routing
profile.  The reference's ``metal_marlin.eval`` names are available too (``compute_perplexity_sliding_window``,
``compute_perplexity_from_logits``, ``compute_perplexity_wikitext``, ``compute_kl_divergence`` (+ ``_np``), ``KLResult``,
``evaluate_kl_divergence``, ``evaluate_kl_from_paths``, ``load_wikitext2``, ``load_tokenizer``, ``softmax``, ``log_softmax``)."""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Callable, List, Optional, Sequence

import numpy as np
import torch

from .moe_routing import ExpertUsageProfiler, apply_capacity, load_balancing_loss
from .perplexity import compute_perplexity, kl_divergence, quality_report, sliding_window_nll, synthetic_corpus


def softmax(x, axis: int = -1) -> np.ndarray:
    a = np.asarray(x, dtype=np.float64)
    e = np.exp(a - a.max(axis=axis, keepdims=True))
    return e / e.sum(axis=axis, keepdims=True)


def log_softmax(x, axis: int = -1) -> np.ndarray:
    a = np.asarray(x, dtype=np.float64)
    s = a - a.max(axis=axis, keepdims=True)
    return s - np.log(np.exp(s).sum(axis=axis, keepdims=True))


def compute_perplexity_from_logits(logits, targets) -> float:
    """``exp(mean NLL)`` of ``targets [T]`` under ``logits [T, V]`` (row t predicts ``targets[t]``)."""
    lg = torch.as_tensor(np.asarray(logits) if not isinstance(logits, torch.Tensor) else logits).float()
    tg = torch.as_tensor(np.asarray(targets) if not isinstance(targets, torch.Tensor) else targets).long()
    return float(torch.exp(torch.nn.functional.cross_entropy(lg.reshape(-1, lg.shape[-1]), tg.reshape(-1))))


def compute_perplexity_sliding_window(logits_fn: Callable, token_ids: Sequence[int], max_length: int = 2048, stride: int = 512) -> float:
    return compute_perplexity(logits_fn, token_ids, max_length, stride)


def load_tokenizer(path: Optional[str] = None, vocab_size: int = 32000):
    from ..inference.tokenizer import load_tokenizer as _lt
    return _lt(path, vocab_size)


def load_wikitext2(tokenizer=None, max_tokens: Optional[int] = None, vocab_size: int = 32000, split: str = "test") -> List[int]:
    """Token ids of the WikiText-2 ``split`` when a copy is available locally (``$METAL_MARLIN_CALIBRATION_DIR/wikitext2.txt`` or
    ``wikitext2-<split>.txt``; there is no network access here), else a deterministic synthetic corpus of the same size."""
    d = os.environ.get("METAL_MARLIN_CALIBRATION_DIR", "")
    for name in (f"wikitext2-{split}.txt", "wikitext2.txt"):
        p = os.path.join(d, name)
        if d and os.path.isfile(p) and tokenizer is not None:
            ids = list(tokenizer.encode(open(p, encoding="utf-8", errors="ignore").read()))
            return ids[:max_tokens] if max_tokens else ids
    return synthetic_corpus(vocab_size, max_tokens or 8192, seed=0)


def compute_perplexity_wikitext(logits_fn: Callable, tokenizer=None, max_length: int = 2048, stride: int = 512,
                                max_tokens: Optional[int] = 8192, vocab_size: int = 32000) -> float:
    return compute_perplexity(logits_fn, load_wikitext2(tokenizer, max_tokens, vocab_size), max_length, stride)


@dataclass
class KLResult:
    kl_mean: float
    kl_max: float
    top1_agreement: float
    num_tokens: int


def compute_kl_divergence(ref_logits, test_logits) -> KLResult:
    """Token-wise ``KL(ref || test)`` of two logit tensors ``[T, V]``."""
    a = torch.as_tensor(np.asarray(ref_logits) if not isinstance(ref_logits, torch.Tensor) else ref_logits).double()
    b = torch.as_tensor(np.asarray(test_logits) if not isinstance(test_logits, torch.Tensor) else test_logits).double()
    la, lb = torch.log_softmax(a, -1), torch.log_softmax(b, -1)
    kl = (la.exp() * (la - lb)).sum(-1)
    return KLResult(float(kl.mean()), float(kl.max()), float((a.argmax(-1) == b.argmax(-1)).double().mean()), int(kl.numel()))


def compute_kl_divergence_np(ref_logits, test_logits) -> float:
    return compute_kl_divergence(ref_logits, test_logits).kl_mean


def evaluate_kl_divergence(ref_fn: Callable, test_fn: Callable, token_ids: Sequence[int], max_length: int = 2048) -> KLResult:
    """Both models over the same windows of ``token_ids`` (``*_fn(ids) -> logits [T, V]``)."""
    r = kl_divergence(ref_fn, test_fn, token_ids, max_length)
    return KLResult(r["kl_mean"], r.get("kl_max", r["kl_mean"]), r.get("top1_agreement", r.get("agreement", 0.0)), int(r.get("positions", len(token_ids))))


def evaluate_kl_from_paths(ref_path: str, test_path: str, token_ids: Optional[Sequence[int]] = None, max_length: int = 512,
                           device: Optional[str] = None) -> KLResult:
    """Load two checkpoints of this engine and compare them on ``token_ids`` (default: a synthetic corpus)."""
    from ..models.mmfp4_causal_lm import MMFP4ForCausalLM
    a, b = MMFP4ForCausalLM.from_pretrained(ref_path, device), MMFP4ForCausalLM.from_pretrained(test_path, device)
    ids = list(token_ids) if token_ids is not None else synthetic_corpus(a.config.vocab_size, 1024, 0)
    return evaluate_kl_divergence(a.forward_logits, b.forward_logits, ids, max_length)


__all__ = ["ExpertUsageProfiler", "apply_capacity", "load_balancing_loss", "compute_perplexity", "kl_divergence", "quality_report",
           "sliding_window_nll", "synthetic_corpus", "KLResult", "compute_kl_divergence", "compute_kl_divergence_np",
           "compute_perplexity_from_logits", "compute_perplexity_sliding_window", "compute_perplexity_wikitext", "evaluate_kl_divergence",
           "evaluate_kl_from_paths", "load_tokenizer", "load_wikitext2", "log_softmax", "softmax"]
