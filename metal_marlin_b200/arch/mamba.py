"""Mamba (selective state space) and Mamba-2 (scalar-decay SSD) layers.

Parity: reference ``metal_marlin/architectures/mamba.py`` / ``mamba2.py``: selective scan
``h_t = exp(dt_t A) h_{t-1} + dt_t B_t x_t``, ``y_t = C_t h_t + D x_t``, causal depthwise conv in front, SiLU gate behind.
``selective_scan_step`` is one launch of ``csrc/recurrent.cu`` on CUDA.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

from .. import ops


def selective_scan(x, dt, A, Bm, Cm, D=None, state: Optional[torch.Tensor] = None):
    """``x, dt [B, T, Di]``, ``A [Di, N]``, ``Bm, Cm [B, T, N]``.  Returns ``(y [B, T, Di], state fp32 [B, Di, N])``."""
    Bsz, T, Di = x.shape
    N = A.shape[1]
    h = torch.zeros(Bsz, Di, N, dtype=torch.float32, device=x.device) if state is None else state.clone().float()
    if x.is_cuda and ops.native_available() and not ops._FORCE_REF and N in (8, 16, 32, 64, 128):
        # one launch over all tokens: the per-channel state stays in registers (csrc/recurrent_scan.cu)
        f = lambda t: t.float().contiguous()
        y = torch.empty(Bsz, T, Di, dtype=torch.float32, device=x.device)
        h = h.contiguous()
        ops.K.mmb200.selective_scan(f(x), f(dt), f(A), f(Bm), f(Cm), None if D is None else f(D), h, y)
        return y.to(x.dtype), h
    ys = torch.empty(Bsz, T, Di, dtype=torch.float32, device=x.device)
    xf, dtf = x.float(), dt.float()
    for t in range(T):
        h = torch.exp(dtf[:, t, :, None] * A.float()[None]) * h + dtf[:, t, :, None] * Bm[:, t].float()[:, None, :] * xf[:, t, :, None]
        ys[:, t] = (h * Cm[:, t].float()[:, None, :]).sum(-1)
    if D is not None:
        ys = ys + D.float() * xf
    return ys.to(x.dtype), h


def selective_scan_step(x, dt, A, Bm, Cm, D, state: torch.Tensor) -> torch.Tensor:
    """One token: ``x, dt [B, Di]``, ``Bm, Cm [B, N]``; ``state`` fp32 ``[B, Di, N]`` updated in place."""
    if x.is_cuda and ops.native_available():
        y = torch.empty(x.shape, dtype=torch.bfloat16, device=x.device)
        ops.K.mmb200.selective_scan_step(x.to(torch.bfloat16).contiguous(), dt.float().contiguous(), A.float().contiguous(),
                                         Bm.float().contiguous(), Cm.float().contiguous(), None if D is None else D.float().contiguous(), state, y)
        return y
    y, h = selective_scan(x[:, None], dt[:, None], A, Bm[:, None], Cm[:, None], D, state)
    state.copy_(h)
    return y[:, 0]


@dataclass
class MambaConfig:
    d_model: int = 256
    d_state: int = 16
    d_conv: int = 4
    expand: int = 2
    dt_rank: Optional[int] = None

    @property
    def d_inner(self) -> int:
        return self.expand * self.d_model

    @property
    def rank(self) -> int:
        return self.dt_rank or max(1, (self.d_model + 15) // 16)


class MambaBlock:
    """Weights as plain tensors (``in_proj [2 Di, d]``, ``conv_w [Di, d_conv]``, ``conv_b``, ``x_proj [rank + 2 N, Di]``,
    ``dt_proj [Di, rank]``, ``dt_bias``, ``A_log [Di, N]``, ``D [Di]``, ``out_proj [d, Di]``)."""

    def __init__(self, cfg: MambaConfig, weights: dict):
        self.cfg, self.w = cfg, weights

    @classmethod
    def random(cls, cfg: MambaConfig, seed: int = 0, device="cpu"):
        g = torch.Generator().manual_seed(seed)
        Di, N, r = cfg.d_inner, cfg.d_state, cfg.rank
        rn = lambda *s: (torch.randn(*s, generator=g) * 0.05).to(device)
        w = {"in_proj": rn(2 * Di, cfg.d_model), "conv_w": rn(Di, cfg.d_conv), "conv_b": rn(Di), "x_proj": rn(r + 2 * N, Di),
             "dt_proj": rn(Di, r), "dt_bias": rn(Di), "A_log": torch.log(torch.arange(1, N + 1).float()).repeat(Di, 1).to(device),
             "D": torch.ones(Di, device=device), "out_proj": rn(cfg.d_model, Di)}
        return cls(cfg, w)

    def _ssm_inputs(self, xc):
        w, N, r = self.w, self.cfg.d_state, self.cfg.rank
        proj = xc @ w["x_proj"].t()
        dt = F.softplus(proj[..., :r] @ w["dt_proj"].t() + w["dt_bias"])
        return dt, proj[..., r:r + N], proj[..., r + N:]

    def forward(self, u: torch.Tensor, state=None):
        """``u [B, T, d]`` -> ``(y [B, T, d], (conv_state [B, Di, d_conv - 1], ssm_state [B, Di, N]))``."""
        w, cfg = self.w, self.cfg
        xz = u.float() @ w["in_proj"].t()
        x, z = xz.chunk(2, -1)
        conv_in = x.transpose(1, 2)
        if state is not None:
            conv_in = torch.cat([state[0], conv_in], -1)
        else:
            conv_in = F.pad(conv_in, (cfg.d_conv - 1, 0))
        xc = F.silu(F.conv1d(conv_in, w["conv_w"].unsqueeze(1), w["conv_b"], groups=cfg.d_inner)).transpose(1, 2)
        dt, Bm, Cm = self._ssm_inputs(xc)
        y, h = selective_scan(xc, dt, -torch.exp(w["A_log"]), Bm, Cm, w["D"], None if state is None else state[1])
        out = (y * F.silu(z)) @ w["out_proj"].t()
        return out.to(u.dtype), (conv_in[..., -(cfg.d_conv - 1):].contiguous(), h)

    def step(self, u: torch.Tensor, state):
        """One token ``u [B, d]`` with the state of :meth:`forward`."""
        y, st = self.forward(u[:, None], state)
        return y[:, 0], st


def mamba2_scan(x, dt, A, Bm, Cm, D=None, state=None):
    """Mamba-2 SSD recurrence with one scalar decay per head: ``x [B, T, H, P]``, ``dt [B, T, H]``, ``A [H]`` (negative),
    ``Bm, Cm [B, T, N]`` shared over heads.  State ``[B, H, P, N]``."""
    B, T, H, P = x.shape
    N = Bm.shape[-1]
    h = torch.zeros(B, H, P, N, dtype=torch.float32, device=x.device) if state is None else state.clone().float()
    ys = torch.empty(B, T, H, P, dtype=torch.float32, device=x.device)
    for t in range(T):
        dA = torch.exp(dt[:, t].float() * A.float())[..., None, None]
        h = dA * h + (dt[:, t].float()[..., None] * x[:, t].float())[..., None] * Bm[:, t].float()[:, None, None, :]
        ys[:, t] = (h * Cm[:, t].float()[:, None, None, :]).sum(-1)
    if D is not None:
        ys = ys + D.float()[None, None, :, None] * x.float()
    return ys.to(x.dtype), h
