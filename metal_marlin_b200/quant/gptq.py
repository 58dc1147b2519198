"""GPTQ and MR-GPTQ weight quantization (second-order, error-compensating) for the group formats of this engine.

Parity: reference ``metal_marlin/gptq.py`` / ``gptq_fp4.py`` / ``gptq_accelerated.py`` (column-wise quantization
with Cholesky-inverse Hessian updates, damping, block size 128, act-order) and ``metal_marlin/mr_gptq.py``
(``:68`` config, ``:164`` Hessian handling, ``:400`` block-Hadamard rotation, ``:620`` kurtosis gating, ``:686``
per-layer loop, ``:974`` stacked-expert tensors, ``:2420`` resumable state).  The Hessian factorisations and the
between-block updates are torch linear algebra on whatever device the tensors are on; on a GPU the column-serial loop
inside a block is one launch of ``csrc/quantizer.cu`` (a warp per weight row, bit-identical to the loop written here).
The output is codes + group scales in the same form the round-to-nearest quantizers produce, so the packers and
checkpoint writers are shared.
"""
from __future__ import annotations

import json
import os
from dataclasses import asdict, dataclass, field
from typing import Callable, Dict, Iterable, List, Optional, Tuple

import torch

from .._compat import E2M1_VALUES, NF4_VALUES
from . import hadamard as had
from .rtn import QuantizedTensor


@dataclass
class GPTQConfig:
    fmt: str = "fp4"                 # fp4 | int4 | nf4 | int8 | int3 | int2
    group_size: int = 128
    block_size: int = 128            # columns updated lazily together
    damp: float = 0.01               # fraction of mean(diag(H)) added to the diagonal
    act_order: bool = False          # quantize columns in order of decreasing Hessian diagonal (static groups)
    symmetric: bool = True           # integer formats: symmetric grid


def _grid(fmt: str, device) -> Tuple[torch.Tensor, float]:
    """Sorted representable values of the format (before scaling) and the value the group absmax maps to."""
    if fmt == "fp4":
        v = torch.tensor(sorted(set(E2M1_VALUES)), dtype=torch.float32, device=device)
        return v, 6.0
    if fmt == "nf4":
        return torch.tensor(sorted(NF4_VALUES), dtype=torch.float32, device=device), 1.0
    bits = {"int8": 8, "int4": 4, "int3": 3, "int2": 2}[fmt]
    q = 2 ** (bits - 1) - 1
    return torch.arange(-q, q + 1, dtype=torch.float32, device=device), float(q)


def _nearest(x: torch.Tensor, grid: torch.Tensor) -> torch.Tensor:
    idx = torch.bucketize(x, (grid[1:] + grid[:-1]) / 2)
    return grid[idx]


def group_scales(w: torch.Tensor, group_size: int, top: float) -> torch.Tensor:
    out_f, in_f = w.shape
    return (w.reshape(out_f, in_f // group_size, group_size).abs().amax(-1) / top).clamp_min(1e-12)


def gptq_quantize(w: torch.Tensor, H: torch.Tensor, cfg: Optional[GPTQConfig] = None) -> Tuple[torch.Tensor, torch.Tensor, Dict]:
    """Quantize ``w [out, in]`` given the input Hessian ``H = sum x x^T [in, in]``.

    Returns ``(w_q fp32 [out, in] - the de-quantized result, scales [out, in / group], stats)``.  Scales are the
    fp16-rounded values that go into the checkpoint, so ``w_q / scale`` lies exactly on the format's grid."""
    cfg = cfg or GPTQConfig()
    dev = w.device
    W = w.to(torch.float32).clone()
    out_f, in_f = W.shape
    gs = cfg.group_size if in_f % cfg.group_size == 0 else in_f
    grid, top = _grid(cfg.fmt, dev)
    H = H.to(torch.float32).clone()
    dead = torch.diag(H) == 0
    H[dead, dead] = 1.0
    W[:, dead] = 0.0
    # static groups: scales from the original weights, one per (row, contiguous group)
    scales = group_scales(W, gs, top).to(torch.float16).to(torch.float32)
    perm = torch.argsort(torch.diag(H), descending=True) if cfg.act_order else torch.arange(in_f, device=dev)
    inv_perm = torch.argsort(perm)
    W = W[:, perm]
    H = H[perm][:, perm]
    col_scale = scales[:, (perm // gs)]                                # scale of every (row, permuted column)
    H += torch.eye(in_f, device=dev) * cfg.damp * torch.diag(H).mean()
    L = torch.linalg.cholesky(H)
    Hinv = torch.linalg.cholesky(torch.cholesky_inverse(L), upper=True)
    Q = torch.zeros_like(W)
    err_total = 0.0
    from .. import ops
    if ops.gptq_block_ok(W, cfg.block_size, grid.numel()):
        # on the GPU the column loop of a block is one kernel launch (a warp per row), same roundings as the loop below
        col_scale, Hrows = col_scale.contiguous(), Hinv.contiguous()     # the kernel reads rows of the factor
        err_rows = torch.zeros(out_f, dtype=torch.float32, device=dev)
        for i1 in range(0, in_f, cfg.block_size):
            i2 = min(i1 + cfg.block_size, in_f)
            E1 = ops.gptq_block(W, Q, Hrows, col_scale, grid, err_rows, i1, i2)
            W[:, i2:] -= E1 @ Hinv[i1:i2, i2:]
        return Q[:, inv_perm], scales, {"sq_err": float(err_rows.sum()), "act_order": cfg.act_order, "group_size": gs}
    for i1 in range(0, in_f, cfg.block_size):
        i2 = min(i1 + cfg.block_size, in_f)
        W1 = W[:, i1:i2].clone()
        E1 = torch.zeros_like(W1)
        Hi = Hinv[i1:i2, i1:i2]
        for i in range(i2 - i1):
            wcol = W1[:, i]
            s = col_scale[:, i1 + i]
            q = _nearest(wcol / s, grid) * s
            Q[:, i1 + i] = q
            d = wcol - q                  # taken before the update below, which also rewrites column i (wcol is a view)
            e = d / Hi[i, i]
            err_total += float((d ** 2).sum())
            W1[:, i:] -= e.unsqueeze(1) * Hi[i, i:].unsqueeze(0)
            E1[:, i] = e
        W[:, i2:] -= E1 @ Hinv[i1:i2, i2:]
    Q = Q[:, inv_perm]
    return Q, scales, {"sq_err": err_total, "act_order": cfg.act_order, "group_size": gs}


def to_quantized_tensor(w_q: torch.Tensor, scales: torch.Tensor, fmt: str, group_size: int) -> QuantizedTensor:
    """Codes for a GPTQ result (``w_q / scale`` is on the grid) in the form the packers take."""
    out_f, in_f = w_q.shape
    gs = group_size if in_f % group_size == 0 else in_f
    norm = w_q.reshape(out_f, in_f // gs, gs) / scales.to(torch.float32).unsqueeze(-1)
    if fmt == "fp4":
        table = torch.tensor(E2M1_VALUES, dtype=torch.float32, device=w_q.device)
        mag = (norm.abs().unsqueeze(-1) - table[:8]).abs().argmin(-1)
        codes = (mag | ((norm < 0) & (mag > 0)).long() << 3).to(torch.uint8).reshape(out_f, in_f)
        return QuantizedTensor(codes, scales.to(torch.float16), None, "fp4", gs, 4)
    if fmt == "nf4":
        table = torch.tensor(NF4_VALUES, dtype=torch.float32, device=w_q.device)
        codes = (norm.unsqueeze(-1) - table).abs().argmin(-1).to(torch.uint8).reshape(out_f, in_f)
        return QuantizedTensor(codes, scales.to(torch.float16), None, "nf4", gs, 4)
    bits = {"int8": 8, "int4": 4, "int3": 3, "int2": 2}[fmt]
    zp = 2 ** (bits - 1) - 1
    codes = (torch.round(norm) + zp).clamp(0, 2 ** bits - 1).to(torch.uint8).reshape(out_f, in_f)
    zeros = torch.full_like(scales, float(zp), dtype=torch.float16)
    return QuantizedTensor(codes, scales.to(torch.float16), zeros, fmt, gs, bits)


# ------------------------------------------------------------------------------------------ MR-GPTQ
@dataclass
class MRGPTQConfig(GPTQConfig):
    hadamard_block: int = 128        # rotation block (<= group size keeps groups aligned with rotation blocks)
    kurtosis_threshold: float = 1.0  # rotate only layers whose mean excess kurtosis exceeds this
    force_rotation: Optional[bool] = None


def mr_gptq_quantize(w: torch.Tensor, H: Optional[torch.Tensor], cfg: Optional[MRGPTQConfig] = None):
    """Block-Hadamard rotation (gated by weight kurtosis) followed by GPTQ (or round-to-nearest when no Hessian is
    given).  Returns ``(w_q, scales, stats)``; when ``stats['rotated']`` the result lives in the rotated basis
    and the runtime must apply ``block_hadamard(x, stats['hadamard_block'])`` to the layer input."""
    cfg = cfg or MRGPTQConfig()
    in_f = w.shape[1]
    k = float(had.kurtosis(w).mean())
    rotate = cfg.force_rotation if cfg.force_rotation is not None else (k > cfg.kurtosis_threshold)
    block = cfg.hadamard_block
    rotate = bool(rotate and in_f % block == 0)
    W = had.rotate_weight(w.to(torch.float32), block) if rotate else w.to(torch.float32)
    if H is None:
        H = torch.eye(in_f, device=w.device)
    elif rotate:
        H = had.rotate_hessian(H, block)
    wq, scales, stats = gptq_quantize(W, H, cfg)
    stats.update({"rotated": rotate, "hadamard_block": block if rotate else 0, "kurtosis": k})
    return wq, scales, stats


def quantize_stacked_experts(w: torch.Tensor, hessians: Optional[List[Optional[torch.Tensor]]], cfg: MRGPTQConfig):
    """``w [E, out, in]``: every expert with its own Hessian (experts that saw no calibration tokens fall back to
    round-to-nearest through an identity Hessian)."""
    outs = [mr_gptq_quantize(w[e], None if hessians is None else hessians[e], cfg) for e in range(w.shape[0])]
    return torch.stack([o[0] for o in outs]), torch.stack([o[1] for o in outs]), [o[2] for o in outs]


class ResumableState:
    """Per-tensor progress record so an interrupted quantization run continues where it stopped
    (``<out_dir>/quantize_state.json``; tensors already written are skipped)."""

    def __init__(self, out_dir: str):
        self.path = os.path.join(out_dir, "quantize_state.json")
        self.done: Dict[str, Dict] = {}
        if os.path.exists(self.path):
            with open(self.path) as f:
                self.done = json.load(f).get("done", {})

    def is_done(self, name: str) -> bool:
        return name in self.done

    def mark(self, name: str, stats: Dict):
        self.done[name] = {k: (v if isinstance(v, (int, float, bool, str)) else str(v)) for k, v in stats.items()}
        tmp = self.path + ".tmp"
        with open(tmp, "w") as f:
            json.dump({"done": self.done}, f)
        os.replace(tmp, self.path)
