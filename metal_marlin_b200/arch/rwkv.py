"""RWKV v5 / v6 time-mix recurrences (WKV).

Per head with state ``S [dk, dv]``:  ``o_t = r_t (S + (u * k_t) v_t^T)``;  ``S <- diag(w_t) S + k_t v_t^T`` where ``w`` is a
fixed per-channel decay in v5 and a data-dependent decay in v6.  Parity: reference ``metal_marlin/architectures/rwkv.py``.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops

_WKV_DK = (16, 32, 64, 128)


def _wkv_native(r, k, v, w, u, state):
    """One launch over all tokens (``csrc/recurrent_scan.cu``): the state stays in registers between tokens."""
    B, T, H, dk = r.shape
    dv = v.shape[-1]
    S = torch.zeros(B, H, dk, dv, dtype=torch.float32, device=r.device) if state is None else state.clone().float().contiguous()
    out = torch.empty(B, T, H, dv, dtype=torch.float32, device=r.device)
    f = lambda t: t.float().contiguous()
    ops.K.mmb200.wkv_scan(f(r), f(k), f(v), f(w), f(u), S, out)
    return out.to(v.dtype), S


def wkv5(r, k, v, w, u, state: Optional[torch.Tensor] = None):
    """``r, k [B, T, H, dk]``, ``v [B, T, H, dv]``, ``w, u [H, dk]`` (``w`` in (0, 1): per-channel decay)."""
    if r.is_cuda and ops.native_available() and not ops._FORCE_REF and r.shape[-1] in _WKV_DK and v.shape[-1] <= 1024:
        return _wkv_native(r, k, v, w, u, state)
    return wkv6(r, k, v, w[None, None].expand(r.shape[0], r.shape[1], -1, -1), u, state)


def wkv6(r, k, v, w, u, state: Optional[torch.Tensor] = None):
    """Same with a decay ``w [B, T, H, dk]`` per token."""
    if r.is_cuda and ops.native_available() and not ops._FORCE_REF and r.shape[-1] in _WKV_DK and v.shape[-1] <= 1024 and w.dim() == 4 \
            and w.is_contiguous():
        return _wkv_native(r, k, v, w, u, state)
    B, T, H, dk = r.shape
    dv = v.shape[-1]
    S = torch.zeros(B, H, dk, dv, dtype=torch.float32, device=r.device) if state is None else state.clone().float()
    out = torch.empty(B, T, H, dv, dtype=torch.float32, device=r.device)
    for t in range(T):
        kv = torch.einsum("bhk,bhv->bhkv", k[:, t].float(), v[:, t].float())
        out[:, t] = torch.einsum("bhk,bhkv->bhv", r[:, t].float(), S + u.float()[None, :, :, None] * kv)
        S = w[:, t].float()[..., None] * S + kv
    return out.to(v.dtype), S
