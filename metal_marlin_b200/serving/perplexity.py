"""Chunked perplexity of a text under the served model.
Parity: reference ``metal_marlin/serving/perplexity.py:39`` (``compute_perplexity``: chunk_size 100 tokens,
per-chunk perplexities, mean loss)."""
from __future__ import annotations

import math
from typing import Dict, List


def compute_perplexity(pipeline, text: str, chunk_size: int = 100, include_token_ppls: bool = False) -> Dict:
    ids = pipeline.encode(text)
    if len(ids) < 2:
        raise ValueError("text is too short to score (need at least 2 tokens)")
    nlls: List[float] = []
    chunk_ppls: List[float] = []
    # every chunk is scored with its own context only, like the reference; one token of overlap gives
    # each chunk boundary token a conditioning token
    for s in range(0, len(ids) - 1, chunk_size):
        chunk = ids[s:s + chunk_size + 1]
        if len(chunk) < 2:
            break
        nll = pipeline.token_nll(chunk).tolist()
        nlls.extend(nll)
        chunk_ppls.append(math.exp(min(50.0, sum(nll) / len(nll))))
    loss = sum(nlls) / len(nlls)
    out = {"perplexity": math.exp(min(50.0, loss)), "tokens": len(nlls), "loss": loss, "chunk_perplexities": chunk_ppls,
           "chunk_size": chunk_size}
    if include_token_ppls:
        out["token_ppls"] = [math.exp(min(50.0, x)) for x in nlls]
    return out
