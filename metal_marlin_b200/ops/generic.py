"""Weights that are not in the FP4 tile layout (trellis, INT4 / INT8 / FP8 / NF4 layers): the op layer runs them
through their own matmul with the fused prologue / epilogue pieces as separate steps.

A generic weight is any object with ``in_features``, ``out_features``, ``__call__(x2d) -> bf16 [M, out]`` and
``dequantize(dtype)``.  ``CatWeight`` stacks such weights along the output axis (fused q_a|kv_a, q|k|v, gate|up);
``GenericExpertBank`` holds per-expert gate|up and down projections (routed experts first, shared experts last).
Parity: the reference's trellis model runs on exactly this kind of layer object (``metal_marlin/trellis/linear.py:50``
``TrellisLinear``, ``metal_marlin/trellis/moe.py:131``).
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch
import torch.nn.functional as F


class CatWeight:
    is_generic = True

    def __init__(self, parts: Sequence):
        self.parts = list(parts)
        self.in_features = parts[0].in_features
        self.out_features = sum(p.out_features for p in parts)
        self.names = None

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        return torch.cat([p(x) for p in self.parts], -1)

    def dequantize(self, dtype=torch.float32) -> torch.Tensor:
        return torch.cat([p.dequantize(dtype) for p in self.parts], 0)


class GenericExpertBank:
    """``gate_up[e]`` maps ``[M, H] -> [M, 2 * I_e]`` (gate rows then up rows), ``down[e]`` maps ``[M, I_e] -> [M, H]``."""
    is_generic = True

    def __init__(self, gate_up: List, down: List):
        self.gate_up, self.down = gate_up, down
        self.num_experts = len(gate_up)
        self.in_features = gate_up[0].in_features
        self.out_features = gate_up[0].out_features
        self.names = None


def is_generic(w) -> bool:
    return getattr(w, "is_generic", False)


def linear(x, W, *, delta=None, norm_w=None, eps=1e-6, resid_out=None, act=0, bias=None, out_add=None, out=None):
    from . import rmsnorm
    xin = x[:, : W.in_features]
    if norm_w is not None:
        xin = rmsnorm(xin, norm_w, eps, delta=None if delta is None else delta[:, : W.in_features], resid_out=resid_out)
    elif delta is not None:
        xin = (xin.to(torch.float32) + delta[:, : W.in_features].to(torch.float32)).to(torch.bfloat16)
        if resid_out is not None:
            resid_out.copy_(xin)
    y = W(xin.contiguous()).to(torch.float32)
    if bias is not None:
        y = y + bias.to(torch.float32)
    if act == 1:
        half = W.out_features // 2
        y = F.silu(y[:, :half]) * y[:, half:]
    if out_add is not None:
        y = y + out_add.to(torch.float32)
    y = y.to(torch.bfloat16)
    if out is not None:
        out.copy_(y)
        return out
    return y


TRELLIS_MOE_MAX_T = 16      # decode-size batches run the routed experts in two device-side launches


def _trellis_parts(bank: GenericExpertBank, n_routed: int):
    """(gate, up, down) TrellisLinear triples of the routed experts, or None if the bank is not uniformly trellis."""
    out = []
    for e in range(n_routed):
        gu, dn = bank.gate_up[e], bank.down[e]
        parts = getattr(gu, "parts", None)
        if parts is None or len(parts) != 2 or not all(hasattr(p, "codes") and hasattr(p, "su") for p in (*parts, dn)):
            return None
        if any(p.bias is not None or p.group_size % 16 for p in (*parts, dn)):
            return None
        out.append((parts[0], parts[1], dn))
    return out


def _trellis_desc(bank: GenericExpertBank, n_routed: int, device):
    """Device table ``int64 [n_routed * 3, 6]`` of the experts' matrices in the layout of ``MmbTrellisMat``."""
    cached = getattr(bank, "_trellis_desc", None)
    if cached is not None and cached[0] == n_routed:
        return cached[1]
    trip = _trellis_parts(bank, n_routed)
    desc = None
    if trip is not None:
        I, H = trip[0][0].out_features, trip[0][0].in_features
        ok = all(g.out_features == I and u.out_features == I and d.in_features == I and d.out_features == H and g.in_features == H
                 for g, u, d in trip) and I % 16 == 0 and H % 16 == 0
        if ok:
            rows = []
            for tr in trip:
                for m in tr:
                    rows.append([m.codes.data_ptr(), m.scales.data_ptr(), m.su.data_ptr(), m.sv.data_ptr(),
                                 m.out_features | (m.in_features << 32), m.bits | (m.group_size << 32)])
            desc = (torch.tensor(rows, dtype=torch.int64).to(device), H, I)
    bank._trellis_desc = (n_routed, desc)
    return desc


def ops_no_tc() -> bool:
    from . import NO_TCGEN05
    return NO_TCGEN05


def moe_forward(x, bank: GenericExpertBank, ids, weights, *, n_shared=0, shared_base=0, norm_w=None, eps=1e-6, out_add=None):
    """Routed + shared experts on generic (trellis, codebook, dense) weights.  Decode-size batches on trellis banks run the
    routed experts in two launches that read the expert ids from device memory (mixed bits per expert and matrix; no
    host synchronization, so the step can be graph captured); otherwise the experts that received tokens are looped over on
    the host."""
    from . import K, _use_native, rmsnorm
    xin = rmsnorm(x, norm_w, eps) if norm_w is not None else x
    T = x.shape[0]
    n_routed = shared_base if n_shared else bank.num_experts
    desc = _trellis_desc(bank, n_routed, x.device) if (_use_native(x) and T <= TRELLIS_MOE_MAX_T and x.dtype == torch.bfloat16) else None
    if desc is not None:
        mats, H, I = desc
        topk = ids.shape[1]
        h = torch.empty(T * topk, I, dtype=torch.bfloat16, device=x.device)
        y = torch.empty(T * topk, H, dtype=torch.float32, device=x.device)
        K.mmb200.trellis_moe(xin if xin.stride(1) == 1 else xin.contiguous(), mats, ids.to(torch.int32).contiguous(),
                             weights.to(torch.float32).contiguous(), h, y, H, I)
        acc = y.view(T, topk, H).sum(1)
        return _finish_shared(acc, xin, bank, n_shared, shared_base, out_add)
    gdesc = _trellis_desc(bank, n_routed, x.device) if (_use_native(x) and x.dtype == torch.bfloat16) else None
    if gdesc is not None and gdesc[1] % 64 == 0 and gdesc[2] % 64 == 0 and not ops_no_tc():
        # prompt-size batches: counting sort by expert and a tile list on the device, then two grouped tensor-core GEMMs that
        # decode the experts' codes (any bit width per expert and matrix) inside their main loops: gate|up with SwiGLU in the
        # epilogue, down with the routing weight; no host synchronisation, no bf16 copy of an expert
        from . import trellis_gemm
        mats, H, I = gdesc
        topk = ids.shape[1]
        n = T * topk
        dev = x.device
        avg = n / max(1, n_routed)
        token_tile = 32 if avg <= 24 else (64 if avg <= 48 else (128 if avg <= 160 else 256))
        max_tiles = (n + token_tile - 1) // token_tile + n_routed
        order = torch.empty(n, dtype=torch.int32, device=dev)
        inv = torch.empty(n, dtype=torch.int32, device=dev)
        t_e = torch.empty(max_tiles, dtype=torch.int32, device=dev)
        t_r0, t_rows = torch.empty_like(t_e), torch.empty_like(t_e)
        n_tiles = torch.empty(1, dtype=torch.int32, device=dev)
        K.mmb200.moe_group(ids.to(torch.int32).reshape(-1).contiguous(), n_routed, token_tile, order, inv, t_e, t_r0, t_rows, n_tiles)
        xs = torch.empty(n, H, dtype=torch.bfloat16, device=dev)
        K.mmb200.moe_gather(xin if xin.stride(1) == 1 else xin.contiguous(), order, xs, topk)
        tiles = (t_e, t_r0, t_rows, n_tiles)
        h = trellis_gemm(xs, mats, 2 * I, H, act=1, first=0, stride=3, tiles=tiles, token_tile=token_tile)
        rs = weights.reshape(-1).to(torch.float32).index_select(0, order.clamp_min(0).long()).contiguous()
        y = trellis_gemm(h, mats, H, I, act=0, first=2, stride=3, tiles=tiles, token_tile=token_tile, row_scale=rs)
        acc = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
        K.mmb200.moe_combine(y, inv, None, None, acc, topk)
        return _finish_shared(acc.to(torch.float32), xin, bank, n_shared, shared_base, out_add)
    acc = torch.zeros(T, bank.down[0].out_features, dtype=torch.float32, device=x.device)
    ids_l = ids.long()
    for e in ids_l.unique().tolist():
        if e < 0:
            continue
        tt, ss = (ids_l == e).nonzero(as_tuple=True)
        gu = bank.gate_up[e](xin[tt].contiguous()).to(torch.float32)
        half = gu.shape[1] // 2
        h = (F.silu(gu[:, :half]) * gu[:, half:]).to(torch.bfloat16)
        acc.index_add_(0, tt, bank.down[e](h).to(torch.float32) * weights[tt, ss].to(torch.float32).unsqueeze(-1))
    return _finish_shared(acc, xin, bank, n_shared, shared_base, out_add)


def _finish_shared(acc, xin, bank, n_shared, shared_base, out_add):
    for j in range(n_shared):
        e = shared_base + j
        if bank.gate_up[e] is None:          # a multi-expert shared MLP kept as one matrix occupies the first slot only
            continue
        gu = bank.gate_up[e](xin.contiguous()).to(torch.float32)
        half = gu.shape[1] // 2
        acc += bank.down[e]((F.silu(gu[:, :half]) * gu[:, half:]).to(torch.bfloat16)).to(torch.float32)
    if out_add is not None:
        acc += out_add.to(torch.float32)
    return acc.to(torch.bfloat16)
