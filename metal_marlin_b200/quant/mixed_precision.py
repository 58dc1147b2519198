"""Mixed-precision presets: which format / group size each tensor class gets, and sensitivity-driven bit
allocation.

Parity: reference ``metal_marlin/mixed_precision.py`` (presets ``dense`` / ``moe`` / ``moe-mtp`` / ``quality`` /
``speed``: attention and shared experts finer groups, routed experts coarser, router / norms / embeddings kept
in 16 bit, MTP head 8 bit) and the adaptive allocation of ``metal_marlin/quantization`` (greedy: spend bits where
the error drop per bit is largest).  Group sizes 32 / 64 / 128 / 256 are all handled by the kernels.
"""
from __future__ import annotations

import re
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple


@dataclass(frozen=True)
class TensorPolicy:
    fmt: str            # "fp4", "int8", ... or "keep" (stay in 16 bit)
    group_size: int = 128


_KEEP = TensorPolicy("keep", 0)
_RULES: Dict[str, List[Tuple[str, TensorPolicy]]] = {
    "dense": [(r"(embed_tokens|lm_head|norm|layernorm)", _KEEP), (r"self_attn\.", TensorPolicy("fp4", 64)),
              (r"mlp\.", TensorPolicy("fp4", 128))],
    "moe": [(r"(embed_tokens|lm_head|norm|layernorm|mlp\.gate\.|router)", _KEEP), (r"self_attn\.", TensorPolicy("fp4", 64)),
            (r"shared_experts?\.", TensorPolicy("fp4", 64)), (r"experts\.", TensorPolicy("fp4", 128)), (r"mlp\.", TensorPolicy("fp4", 128))],
    "moe-mtp": [(r"(embed_tokens|lm_head|norm|layernorm|mlp\.gate\.|router)", _KEEP), (r"(mtp|nextn|eh_proj)", TensorPolicy("int8", 128)),
                (r"self_attn\.", TensorPolicy("fp4", 64)), (r"shared_experts?\.", TensorPolicy("fp4", 64)),
                (r"experts\.", TensorPolicy("fp4", 128)), (r"mlp\.", TensorPolicy("fp4", 128))],
    "quality": [(r"(embed_tokens|lm_head|norm|layernorm|mlp\.gate\.|router)", _KEEP), (r"self_attn\.", TensorPolicy("int8", 128)),
                (r"shared_experts?\.", TensorPolicy("fp4", 32)), (r"experts\.", TensorPolicy("fp4", 64)), (r"mlp\.", TensorPolicy("fp4", 32))],
    "speed": [(r"(embed_tokens|norm|layernorm|mlp\.gate\.|router)", _KEEP), (r"lm_head", TensorPolicy("fp4", 128)),
              (r".", TensorPolicy("fp4", 256))],
}
PRESETS = tuple(_RULES)


def policy_for(name: str, preset: str = "dense") -> TensorPolicy:
    try:
        rules = _RULES[preset]
    except KeyError:
        raise ValueError(f"unknown mixed-precision preset {preset!r}; known: {PRESETS}") from None
    for pat, pol in rules:
        if re.search(pat, name):
            return pol
    return TensorPolicy("fp4", 128)


def allocate_bits(sensitivity: Dict[str, Dict[int, float]], sizes: Dict[str, int], target_bpw: float,
                  choices: Sequence[int] = (2, 3, 4, 5, 6, 8)) -> Dict[str, int]:
    """Greedy bit allocation: ``sensitivity[name][bits]`` is the error of tensor ``name`` at ``bits``; start every
    tensor at the smallest choice and repeatedly upgrade the tensor with the largest error drop per extra bit of
    storage until the average bits-per-weight reaches ``target_bpw``."""
    choices = sorted(choices)
    alloc = {n: choices[0] for n in sensitivity}
    total = sum(sizes.values())
    used = sum(sizes[n] * alloc[n] for n in alloc)
    while True:
        best, best_gain = None, 0.0
        for n, b in alloc.items():
            i = choices.index(b)
            if i + 1 >= len(choices):
                continue
            nb = choices[i + 1]
            cost = sizes[n] * (nb - b)
            if used + cost > target_bpw * total:
                continue
            gain = (sensitivity[n][b] - sensitivity[n][nb]) / cost
            if gain > best_gain:
                best, best_gain = (n, nb, cost), gain
        if best is None:
            return alloc
        alloc[best[0]] = best[1]
        used += best[2]
