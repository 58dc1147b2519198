"""Rotary position embeddings: plain, linear / dynamic-NTK scaling and YaRN, plus the latent (MLA) variant.

Parity: reference ``metal_marlin/rope.py`` — ``YaRNConfig.from_hf_config`` (``:133``), the inverse-frequency
ramp (``:250``), the attention scale ``mscale`` (``:327``), cos/sin caches (``:386``) and the MLA latent RoPE
(``:923``).  The CUDA kernels take ``inv_freq`` and ``mscale`` computed here (``csrc/elementwise.cu`` rope
kernels, the MLA prologue in ``csrc/attention_decode.cu``); this module is also the CPU oracle for them.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Tuple

import torch


@dataclass
class YaRNConfig:
    original_max_position: int = 4096
    scale_factor: float = 1.0
    beta_fast: float = 32.0
    beta_slow: float = 1.0
    mscale: float = 1.0
    mscale_all_dim: float = 0.0
    rope_theta: float = 10000.0

    @classmethod
    def from_hf_config(cls, cfg) -> Optional["YaRNConfig"]:
        """Build from a HF config (object or dict); ``None`` when the model does not use YaRN."""
        get = (lambda k, d=None: cfg.get(k, d)) if isinstance(cfg, dict) else (lambda k, d=None: getattr(cfg, k, d))
        rs = get("rope_scaling") or get("rope_parameters")
        if not rs or (rs.get("type") or rs.get("rope_type")) != "yarn":
            return None
        return cls(original_max_position=int(rs.get("original_max_position_embeddings", get("max_position_embeddings", 4096))),
                   scale_factor=float(rs.get("factor", 1.0)), beta_fast=float(rs.get("beta_fast", 32.0)),
                   beta_slow=float(rs.get("beta_slow", 1.0)), mscale=float(rs.get("mscale", 1.0)),
                   mscale_all_dim=float(rs.get("mscale_all_dim", 0.0)), rope_theta=float(get("rope_theta", 10000.0)))


def yarn_get_mscale(scale: float, mscale: float = 1.0) -> float:
    return 1.0 if scale <= 1.0 else 0.1 * mscale * math.log(scale) + 1.0


def _correction_dim(num_rot: float, dim: int, base: float, max_pos: int) -> float:
    return dim * math.log(max_pos / (num_rot * 2 * math.pi)) / (2 * math.log(base))


def yarn_inv_freq(dim: int, cfg: YaRNConfig) -> Tuple[torch.Tensor, float]:
    """NTK-by-parts: low-frequency dimensions are interpolated (divided by the factor), high-frequency ones keep
    their wavelength, with a linear ramp between ``beta_slow`` and ``beta_fast`` rotations.  Returns
    ``(inv_freq fp32 [dim/2], mscale)`` where ``mscale`` multiplies cos and sin."""
    base = cfg.rope_theta
    pos_freq = base ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim)
    extra, inter = 1.0 / pos_freq, 1.0 / (cfg.scale_factor * pos_freq)
    low = max(math.floor(_correction_dim(cfg.beta_fast, dim, base, cfg.original_max_position)), 0)
    high = min(math.ceil(_correction_dim(cfg.beta_slow, dim, base, cfg.original_max_position)), dim - 1)
    if low == high:
        high += 0.001
    ramp = ((torch.arange(dim // 2, dtype=torch.float32) - low) / (high - low)).clamp(0, 1)
    extra_mask = 1.0 - ramp
    inv = inter * (1 - extra_mask) + extra * extra_mask
    if cfg.mscale_all_dim:
        m = yarn_get_mscale(cfg.scale_factor, cfg.mscale) / yarn_get_mscale(cfg.scale_factor, cfg.mscale_all_dim)
    else:
        m = yarn_get_mscale(cfg.scale_factor, cfg.mscale)
    return inv.contiguous(), float(m)


def rope_inv_freq(dim: int, theta: float = 10000.0, scaling: Optional[dict] = None,
                  max_position: int = 4096) -> Tuple[torch.Tensor, float]:
    """``(inv_freq, mscale)`` for ``rope_scaling`` types none / linear / dynamic / yarn."""
    inv = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))
    if not scaling:
        return inv, 1.0
    kind = scaling.get("type") or scaling.get("rope_type") or "default"
    factor = float(scaling.get("factor", 1.0))
    if kind in ("default", "none"):
        return inv, 1.0
    if kind == "linear":
        return inv / factor, 1.0
    if kind == "dynamic":
        t = theta * ((factor * max_position / scaling.get("original_max_position_embeddings", max_position)) - (factor - 1)) ** (dim / (dim - 2))
        return 1.0 / (t ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim)), 1.0
    if kind == "yarn":
        return yarn_inv_freq(dim, YaRNConfig(
            original_max_position=int(scaling.get("original_max_position_embeddings", max_position)), scale_factor=factor,
            beta_fast=float(scaling.get("beta_fast", 32.0)), beta_slow=float(scaling.get("beta_slow", 1.0)),
            mscale=float(scaling.get("mscale", 1.0)), mscale_all_dim=float(scaling.get("mscale_all_dim", 0.0)), rope_theta=theta))
    raise ValueError(f"unsupported rope scaling type {kind!r}")


def cos_sin_cache(inv_freq: torch.Tensor, max_position: int, mscale: float = 1.0, device=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """fp32 ``[max_position, dim/2]`` tables."""
    pos = torch.arange(max_position, dtype=torch.float32, device=device)
    ang = pos[:, None] * inv_freq.to(device)[None, :]
    return ang.cos() * mscale, ang.sin() * mscale


def apply_rope(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor, *, interleaved: bool = False,
               mscale: float = 1.0, rot_dim: Optional[int] = None) -> torch.Tensor:
    """Rotate the first ``rot_dim`` features of ``x [..., T, H, D]`` (positions ``[T]``).  ``interleaved`` pairs
    ``(2i, 2i+1)`` (GPT-J / GLM style); otherwise ``(i, i + rot/2)`` (NeoX / Llama style)."""
    D = x.shape[-1]
    rot = rot_dim or 2 * inv_freq.numel()
    ang = positions.to(torch.float32)[:, None] * inv_freq.to(x.device)[None, :]
    cos, sin = (ang.cos() * mscale)[:, None, :], (ang.sin() * mscale)[:, None, :]
    xr = x[..., :rot].to(torch.float32)
    if interleaved:
        a, b = xr[..., 0::2], xr[..., 1::2]
        out = torch.stack([a * cos - b * sin, b * cos + a * sin], -1).flatten(-2)
    else:
        a, b = xr[..., : rot // 2], xr[..., rot // 2:]
        out = torch.cat([a * cos - b * sin, b * cos + a * sin], -1)
    return torch.cat([out.to(x.dtype), x[..., rot:]], -1) if rot < D else out.to(x.dtype)


class RotaryEmbedding:
    """Caches ``inv_freq`` / ``mscale`` for a model and rotates q and k.  ``MLARoPE`` semantics (rotating only the
    decoupled ``rope`` slice of an MLA head or latent row) are the ``rot_dim`` / slice arguments."""

    def __init__(self, dim: int, theta: float = 10000.0, scaling: Optional[dict] = None, max_position: int = 4096,
                 interleaved: bool = False):
        self.dim, self.interleaved = dim, interleaved
        self.inv_freq, self.mscale = rope_inv_freq(dim, theta, scaling, max_position)

    def __call__(self, q: torch.Tensor, k: torch.Tensor, positions: torch.Tensor):
        kw = dict(interleaved=self.interleaved, mscale=self.mscale)
        return apply_rope(q, positions, self.inv_freq, **kw), apply_rope(k, positions, self.inv_freq, **kw)

    def rotate_latent(self, latent: torch.Tensor, positions: torch.Tensor, rope_offset: int) -> torch.Tensor:
        """MLA latent rows ``[T, R + dr]``: rotate only the trailing ``dr`` features."""
        head, tail = latent[..., :rope_offset], latent[..., rope_offset:]
        tail = apply_rope(tail.unsqueeze(-2), positions, self.inv_freq, interleaved=self.interleaved, mscale=self.mscale).squeeze(-2)
        return torch.cat([head, tail], -1)
