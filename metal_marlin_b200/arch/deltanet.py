"""Gated DeltaNet (linear attention with the gated delta rule), the recurrent layer of Qwen3.5 / 3.6 hybrid models.

Recurrence per head (state ``S [dk, dv]``):  ``S <- S * exp(g_t)``;  ``m = S^T k_t``;  ``S <- S + k_t ((v_t - m) beta_t)^T``;
``o_t = S^T q_t``.  Parity: reference ``metal_marlin/qwen36_27b_*.py`` / ``kernels/qwen36_27b.py`` (fused DeltaNet decode
path) and the DeltaNet fields of ``metal_marlin/trellis/config.py:75``.  ``gated_delta_step`` is one launch of
``csrc/recurrent.cu`` on CUDA; the chunked form is the prefill path.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn.functional as F

from .. import ops


def gated_delta_rule_recurrent(q, k, v, g, beta, state: Optional[torch.Tensor] = None, scale: Optional[float] = None):
    """Token-by-token reference.  ``q, k [B, T, H, dk]``, ``v [B, T, H, dv]``, ``g, beta [B, T, H]``.  Returns
    ``(o [B, T, H, dv], final state fp32 [B, H, dk, dv])``."""
    B, T, H, dk = q.shape
    dv = v.shape[-1]
    scale = scale if scale is not None else dk ** -0.5
    S = torch.zeros(B, H, dk, dv, dtype=torch.float32, device=q.device) if state is None else state.clone().float()
    out = torch.empty(B, T, H, dv, dtype=torch.float32, device=q.device)
    qf, kf, vf = q.float() * scale, k.float(), v.float()
    for t in range(T):
        S = S * torch.exp(g[:, t].float())[..., None, None]
        m = torch.einsum("bhkv,bhk->bhv", S, kf[:, t])
        d = (vf[:, t] - m) * beta[:, t].float()[..., None]
        S = S + torch.einsum("bhk,bhv->bhkv", kf[:, t], d)
        out[:, t] = torch.einsum("bhkv,bhk->bhv", S, qf[:, t])
    return out.to(v.dtype), S


def gated_delta_rule_chunked(q, k, v, g, beta, state: Optional[torch.Tensor] = None, scale: Optional[float] = None, chunk: int = 64):
    """Chunk-parallel prefill: inside a chunk the delta rule is solved as a lower-triangular system (WY form), across
    chunks the state is carried.  Same result as the recurrence up to rounding."""
    B, T, H, dk = q.shape
    dv = v.shape[-1]
    scale = scale if scale is not None else dk ** -0.5
    S = torch.zeros(B, H, dk, dv, dtype=torch.float32, device=q.device) if state is None else state.clone().float()
    out = torch.empty(B, T, H, dv, dtype=torch.float32, device=q.device)
    if q.is_cuda and ops.native_available() and not ops._FORCE_REF and dk in (16, 32, 64, 128) and dv <= 1024:
        # prompt pass on the device in one launch: every value column's state vector lives in registers while the kernel
        # walks the tokens (csrc/recurrent_scan.cu); the chunk-parallel form below is the CPU / oracle path
        f = lambda t: t.float().contiguous()
        S = S.contiguous()
        ops.K.mmb200.gated_delta_scan(f(q), f(k), f(v), f(g), f(beta), S, out, float(scale))
        return out.to(v.dtype), S
    for c0 in range(0, T, chunk):
        c1 = min(T, c0 + chunk)
        L = c1 - c0
        qc = (q[:, c0:c1].float() * scale).transpose(1, 2)        # [B, H, L, dk]
        kc = k[:, c0:c1].float().transpose(1, 2)
        vc = v[:, c0:c1].float().transpose(1, 2)
        bc = beta[:, c0:c1].float().transpose(1, 2)               # [B, H, L]
        G = torch.cumsum(g[:, c0:c1].float().transpose(1, 2), -1)  # cumulative log decay inside the chunk
        # decay from step j (after its update) to step i (before its read): exp(G_i - G_j)
        decay = torch.exp(G[..., :, None] - G[..., None, :])
        tril = torch.tril(torch.ones(L, L, device=q.device, dtype=torch.bool), -1)
        # u_i = beta_i (v_i - exp(G_i) S0^T k_i - sum_{j<i} exp(G_i - G_j) (k_j . k_i) u_j)
        kk = (kc @ kc.transpose(-1, -2)) * decay
        A = torch.where(tril, kk * bc[..., :, None], torch.zeros_like(kk))
        rhs = bc[..., None] * (vc - torch.exp(G)[..., None] * (kc @ S))
        eye = torch.eye(L, device=q.device)
        U = torch.linalg.solve_triangular(eye + A, rhs, upper=False)
        # o_i = exp(G_i) S0^T q_i + sum_{j<=i} exp(G_i - G_j) (k_j . q_i) u_j
        qk = (qc @ kc.transpose(-1, -2)) * decay
        qk = torch.where(torch.tril(torch.ones(L, L, device=q.device, dtype=torch.bool)), qk, torch.zeros_like(qk))
        oc = torch.exp(G)[..., None] * (qc @ S) + qk @ U
        out[:, c0:c1] = oc.transpose(1, 2)
        # carry: S <- exp(G_L) S0 + sum_j exp(G_L - G_j) k_j u_j^T
        wj = torch.exp(G[..., -1:] - G)                            # [B, H, L]
        S = torch.exp(G[..., -1])[..., None, None] * S + (kc * wj[..., None]).transpose(-1, -2) @ U
    return out.to(v.dtype), S


def gated_delta_step(q, k, v, g, beta, state: torch.Tensor, scale: Optional[float] = None) -> torch.Tensor:
    """One decode token: ``q, k [B, H, dk]``, ``v [B, H, dv]``, ``g, beta [B, H]``; ``state`` fp32 updated in place."""
    dk = q.shape[-1]
    scale = scale if scale is not None else dk ** -0.5
    if q.is_cuda and ops.native_available():
        out = torch.empty_like(v, dtype=torch.bfloat16)
        ops.K.mmb200.gated_delta_step(q.to(torch.bfloat16).contiguous(), k.to(torch.bfloat16).contiguous(), v.to(torch.bfloat16).contiguous(),
                                      g.float().contiguous(), beta.float().contiguous(), state, out, scale)
        return out
    o, S = gated_delta_rule_recurrent(q[:, None], k[:, None], v[:, None], g[:, None], beta[:, None], state, scale)
    state.copy_(S)
    return o[:, 0]


def l2norm(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    return x * torch.rsqrt(x.float().pow(2).sum(-1, keepdim=True) + eps).to(x.dtype)
