"""AWQ: activation-aware per-input-channel scaling searched on a grid before group quantization.

Two levels:

* one matrix (:func:`awq_search`, :func:`awq_quantize`): per-channel scale ``s = mean|x|^alpha``, ``alpha`` searched over a grid
  to minimise the output error on calibration activations; returns the quantized ``W * s`` and ``s`` (the caller owns the
  ``x / s`` side);
* a whole checkpoint (:func:`awq_plan`, :func:`apply_awq_plan`): every group of projections that read the output of one
  RMSNorm shares one scale vector, searched on the sum of their output errors; the projections' input channels are multiplied
  by ``s`` before quantization and the norm's weight is divided by ``s`` (the router of a MoE block, which reads the same
  normalised activation in high precision, gets its columns multiplied by ``s`` as well), so the checkpoint stays a plain
  weights-only checkpoint that every loader runs unchanged - the activation is pre-divided by the norm itself.

Parity: reference ``metal_marlin/awq.py`` (scale search on calibration activations; the scale folded into the weight and its
inverse into the producer of the activation).
"""
from __future__ import annotations

import re
from typing import Callable, Dict, Iterable, Iterator, List, Optional, Tuple

import torch

from .rtn import quantize as rtn_quantize


def awq_search(w: torch.Tensor, x: torch.Tensor, fmt: str = "fp4", group_size: int = 128, n_grid: int = 20) -> Tuple[torch.Tensor, Dict]:
    """``w [out, in]``, calibration activations ``x [n, in]``.  Returns the per-channel scale ``s [in]`` (the layer
    becomes ``(W * s) (x / s)``) and search statistics."""
    W = w.to(torch.float32)
    X = x.to(torch.float32)
    ref = X @ W.t()
    act = X.abs().mean(0).clamp_min(1e-8)
    best, best_err, best_alpha = torch.ones_like(act), float("inf"), 0.0
    for i in range(n_grid + 1):
        alpha = i / n_grid
        s = act.pow(alpha)
        s = s / (s.max() * s.min()).sqrt()
        wq = rtn_quantize(W * s, fmt, group_size).dequantize(torch.float32) / s
        err = float(((X @ wq.t()) - ref).pow(2).mean())
        if err < best_err:
            best, best_err, best_alpha = s, err, alpha
    base = float(((X @ rtn_quantize(W, fmt, group_size).dequantize(torch.float32).t()) - ref).pow(2).mean())
    return best, {"alpha": best_alpha, "mse": best_err, "mse_rtn": base}


def awq_quantize(w: torch.Tensor, x: torch.Tensor, fmt: str = "fp4", group_size: int = 128, n_grid: int = 20):
    """Returns ``(QuantizedTensor of W * s, s, stats)``."""
    s, stats = awq_search(w, x, fmt, group_size, n_grid)
    return rtn_quantize(w.to(torch.float32) * s, fmt, group_size), s, stats


# ---------------------------------------------------------------------------------------------------- whole checkpoints
# (norm tensor suffix, consumers that read its output, high-precision readers that must be compensated)
_GROUPS = (
    ("input_layernorm.weight", (r"self_attn\.(q_proj|k_proj|v_proj|q_a_proj|kv_a_proj_with_mqa)\.weight$",), ()),
    ("post_attention_layernorm.weight", (r"mlp\.(gate_proj|up_proj)\.weight$", r"mlp\.experts\.\d+\.(gate_proj|up_proj)\.weight$",
                                         r"mlp\.shared_experts?\.(gate_proj|up_proj)\.weight$"), (r"mlp\.gate\.weight$",)),
    ("self_attn.q_a_layernorm.weight", (r"self_attn\.q_b_proj\.weight$",), ()),
)


def awq_plan(names: Iterable[str], get_weight: Callable[[str], torch.Tensor], get_inputs: Callable[[str], Optional[torch.Tensor]],
             fmt: str = "fp4", group_size: int = 128, n_grid: int = 10, max_consumers: int = 6) -> Dict[str, Dict]:
    """Scale vectors for every (norm -> projections) group found among ``names`` (HF tensor names).

    ``get_weight(name)`` returns a float matrix, ``get_inputs(name)`` calibration rows of that matrix's input (or ``None``).
    Returns ``{norm name: {"scale": s [in], "consumers": [...], "compensate": [...], "alpha", "mse", "mse_rtn"}}``.  The search
    objective sums the output error over at most ``max_consumers`` of the group's projections (a MoE block has hundreds)."""
    names = list(names)
    by_layer: Dict[str, List[str]] = {}
    for n in names:
        m = re.match(r"(.*\blayers\.\d+\.)", n)
        if m:
            by_layer.setdefault(m.group(1), []).append(n)
    plan: Dict[str, Dict] = {}
    for prefix, members in by_layer.items():
        for norm_suffix, pats, comp_pats in _GROUPS:
            norm = prefix + norm_suffix
            if norm not in members:
                continue
            cons = [n for n in members if any(re.search(p, n[len(prefix):]) for p in pats)]
            comp = [n for n in members if any(re.search(p, n[len(prefix):]) for p in comp_pats)]
            xs = [(n, get_inputs(n)) for n in cons]
            xs = [(n, x) for n, x in xs if x is not None and x.numel()]
            if not cons or not xs:
                continue
            X = torch.cat([x.to(torch.float32) for _, x in xs[:max_consumers]], 0)
            act = X.abs().mean(0).clamp_min(1e-8)
            sample = [n for n, _ in xs[:max_consumers]]
            Ws = [get_weight(n).to(torch.float32) for n in sample]
            gs = group_size if Ws[0].shape[1] % group_size == 0 else 64
            refs = [X @ W.t() for W in Ws]
            norm_ref = sum(float(r.pow(2).mean()) for r in refs)

            def err_of(sv):
                e = 0.0
                for W, r in zip(Ws, refs):
                    wq = rtn_quantize(W * sv, fmt, gs).dequantize(torch.float32) / sv
                    e += float(((X @ wq.t()) - r).pow(2).mean())
                return e / max(norm_ref, 1e-30)

            base = err_of(torch.ones_like(act))
            best, best_err, best_alpha = torch.ones_like(act), base, 0.0
            for i in range(1, n_grid + 1):
                alpha = i / n_grid
                sv = act.pow(alpha)
                sv = sv / (sv.max() * sv.min()).sqrt()
                e = err_of(sv)
                if e < best_err:
                    best, best_err, best_alpha = sv, e, alpha
            plan[norm] = {"scale": best, "consumers": cons, "compensate": comp, "alpha": best_alpha, "mse": best_err, "mse_rtn": base}
    return plan


def apply_awq_plan(tensors: Iterable[Tuple[str, torch.Tensor]], plan: Dict[str, Dict]) -> Iterator[Tuple[str, torch.Tensor]]:
    """Stream ``(name, tensor)`` pairs with the plan applied: norms divided by their scale, consumers' and compensated readers'
    input channels multiplied by it.  The function the model computes is unchanged (up to float rounding)."""
    mul: Dict[str, torch.Tensor] = {}
    for norm, g in plan.items():
        for n in g["consumers"] + g["compensate"]:
            mul[n] = g["scale"]
    for name, t in tensors:
        if name in plan:
            yield name, (t.to(torch.float32) / plan[name]["scale"].to(t.device)).to(t.dtype)
        elif name in mul:
            yield name, (t.to(torch.float32) * mul[name].to(t.device).unsqueeze(0)).to(t.dtype)
        else:
            yield name, t
