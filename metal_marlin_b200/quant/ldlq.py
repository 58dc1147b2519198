"""LDLQ: Hessian-aware quantization to the trellis grid with block error feedback (the quantizer of the EXL3 pipeline).

The input Hessian ``H = X^T X`` is factored block-wise, ``H = L D L^T`` with ``L`` unit block-lower-triangular (16 x 16 identity
blocks on the diagonal).  Input columns are quantized in 16-column blocks from the last to the first; before a block is
rounded to the grid, the rounding error of every block already done is fed back through the matching columns of ``L``:

    target[:, b] = W[:, b] + (W[:, later] - Wq[:, later]) @ L[later, b]

which minimises the proxy error ``tr((W - Wq) H (W - Wq)^T)`` over the order of rounding decisions (with ``L = I`` it is the
plain nearest-grid quantizer).  Each 16 x 16 tile is rounded by a search over its grid sequence; on the uniform scalar grid
with state-independent transition costs the optimal path is the per-element nearest code, which is what runs here (on the
device of the weight: the whole layer is a handful of matrix products).

Parity: reference ``metal_marlin/quantization/ldl_decomp.py:34`` (``block_ldl``), ``:148`` (``ldl_solve``),
``metal_marlin/quantization/ldlq.py:32`` (``compute_group_scales``), ``:166`` (``ldlq_quantize_layer``: bottom-up 16-row blocks,
``prod_cache`` feedback), ``metal_marlin/quantization/viterbi_quant.py:91`` (``quantize_tile_viterbi``), ``:261``
(``quantize_tile_greedy``), ``:295`` (``compute_quantization_error``), ``metal_marlin/quantization/exl3_quantizer.py``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from ..formats.trellis import GRID_SCALE, TrellisWeight, pack_codes

TILE = 16


def block_ldl(H: torch.Tensor, block: int = TILE, damp: float = 0.01) -> Tuple[torch.Tensor, torch.Tensor]:
    """``H = L D L^T`` with unit block-lower-triangular ``L`` and block-diagonal ``D`` (returned as ``[n / block, block, block]``).
    ``H`` is symmetrised and damped (``damp`` x mean diagonal) first; computed in float64 from the Cholesky factor."""
    n = H.shape[0]
    if n % block:
        raise ValueError(f"Hessian size {n} is not a multiple of the block size {block}")
    Hd = H.to(torch.float64)
    Hd = 0.5 * (Hd + Hd.t())
    Hd = Hd + torch.eye(n, dtype=torch.float64, device=H.device) * (damp * Hd.diagonal().mean().clamp_min(1e-12))
    C = torch.linalg.cholesky(Hd)                                   # H = C C^T
    nb = n // block
    Cd = torch.stack([C[i * block:(i + 1) * block, i * block:(i + 1) * block] for i in range(nb)])      # diagonal blocks
    # L = C * blockdiag(Cd)^-1 (unit diagonal blocks); D = Cd Cd^T
    L = C.clone()
    for i in range(nb):
        sl = slice(i * block, (i + 1) * block)
        L[:, sl] = torch.linalg.solve_triangular(Cd[i], C[:, sl].contiguous(), upper=False, left=False)      # C[:, sl] Cd^-1
    D = Cd @ Cd.transpose(1, 2)
    return L, D


def ldl_reconstruct(L: torch.Tensor, D: torch.Tensor) -> torch.Tensor:
    return L @ torch.block_diag(*D) @ L.t()


def compute_group_scales(w: torch.Tensor, bits: int, group_size: int) -> torch.Tensor:
    """Per (output row, input group) scale that maps the group's largest magnitude onto the outermost grid point:
    ``[out, in / group_size]``."""
    out_f, in_f = w.shape
    gmax = (((1 << bits) - 1) / 2.0) * GRID_SCALE
    return (w.view(out_f, in_f // group_size, group_size).abs().amax(-1) / gmax).clamp_min(1e-12)


def quantize_tile_greedy(t: torch.Tensor, scale: torch.Tensor, bits: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Nearest grid code of every element: ``t [..., 16]`` with broadcastable ``scale`` -> ``(codes uint8, de-quantized)``."""
    half = ((1 << bits) - 1) / 2.0
    codes = (t / scale / GRID_SCALE + half).round().clamp_(0, (1 << bits) - 1)
    return codes.to(torch.uint8), (codes - half) * GRID_SCALE * scale


quantize_tile_viterbi = quantize_tile_greedy      # state-independent transition costs: the optimal path is the nearest code


def proxy_error(w: torch.Tensor, wq: torch.Tensor, H: torch.Tensor) -> float:
    """``tr((W - Wq) H (W - Wq)^T) / tr(W H W^T)``: the layer-output error the Hessian predicts, relative."""
    e = (w - wq).to(torch.float64)
    Hd = H.to(torch.float64)
    return float(torch.einsum("oi,ij,oj->", e, Hd, e) / torch.einsum("oi,ij,oj->", w.double(), Hd, w.double()).clamp_min(1e-30))


@dataclass
class LDLQResult:
    weight: TrellisWeight
    dequantized: torch.Tensor         # [out, in] float32, original (unrotated) basis
    proxy_error: float
    mse: float


def ldlq_quantize(w: torch.Tensor, H: Optional[torch.Tensor], bits: int = 4, group_size: int = 128, *, damp: float = 0.01,
                  buf_size_k: int = 128, seed: int = 0, random_signs: bool = True) -> LDLQResult:
    """Quantize ``w [out, in]`` to a trellis tensor of ``bits`` per weight with LDL error feedback against ``H [in, in]``
    (``H = None``: identity, i.e. nearest-grid rounding).  ``in`` must be a multiple of 16 and of ``group_size``."""
    out_f, in_f = w.shape
    if in_f % TILE or in_f % group_size or group_size % TILE:
        raise ValueError("in_features must be a multiple of 16 and of the group size (itself a multiple of 16)")
    dev = w.device
    g = torch.Generator(device="cpu").manual_seed(seed)
    if random_signs:
        su = (torch.randint(0, 2, (in_f,), generator=g).float() * 2 - 1).to(dev)
        sv = (torch.randint(0, 2, (out_f,), generator=g).float() * 2 - 1).to(dev)
    else:
        su, sv = torch.ones(in_f, device=dev), torch.ones(out_f, device=dev)
    wr = (w.float() * sv.view(-1, 1) * su.view(1, -1)).to(torch.float64)          # rotated basis the codes live in
    if H is not None:
        Hr = H.to(dev, torch.float64) * su.view(-1, 1).double() * su.view(1, -1).double()      # the same diagonal rotation
        L, _ = block_ldl(Hr, TILE, damp)
    else:
        Hr, L = None, None
    scales = compute_group_scales(wr.float(), bits, group_size).double()            # [out, ng]
    wq = torch.zeros_like(wr)
    codes = torch.zeros(out_f, in_f, dtype=torch.uint8, device=dev)
    prod = torch.zeros_like(wr)                                                     # feedback carried in from finished spans
    for j in range(in_f, 0, -buf_size_k):
        i = max(0, j - buf_size_k)
        for bj in range(j, i, -TILE):
            bi = bj - TILE
            tgt = wr[:, bi:bj] + prod[:, bi:bj]
            if L is not None and bj < j:                                            # feedback from the blocks of this span already done
                tgt = tgt + (wr[:, bj:j] - wq[:, bj:j]) @ L[bj:j, bi:bj]
            sc = scales[:, bi // group_size].unsqueeze(1)
            c, dq = quantize_tile_greedy(tgt, sc, bits)
            codes[:, bi:bj] = c
            wq[:, bi:bj] = dq
        if L is not None and i > 0:
            prod[:, :i] += (wr[:, i:j] - wq[:, i:j]) @ L[i:j, :i]
    tw = TrellisWeight(pack_codes(codes.cpu(), bits), scales.t().contiguous().float().cpu(), su.cpu(), sv.cpu(), (out_f, in_f))
    deq = (wq.float() * sv.view(-1, 1) * su.view(1, -1))
    pe = proxy_error(wr, wq, Hr) if Hr is not None else float(((wr - wq) ** 2).sum() / (wr ** 2).sum().clamp_min(1e-30))
    return LDLQResult(tw, deq, pe, float(((w.float() - deq) ** 2).mean()))
