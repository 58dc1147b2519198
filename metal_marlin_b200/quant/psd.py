"""Positive-semi-definiteness helpers for the Hessian-based quantizers (GPTQ, MR-GPTQ, trellis LDL).

``gershgorin_is_psd`` is the cheap sufficient test (every Gershgorin disc in the right half plane), ``project_psd`` the
exact repair (eigenvalue clipping), ``damp_until_cholesky`` the usual cheap repair (add multiples of the mean diagonal
until the factorization succeeds).  All run wherever the Hessian lives (``torch.linalg`` on the GPU).

Parity: reference ``metal_marlin/_psd_dispatch.mm`` (Gershgorin PSD check, projection) and ``src/psd_project.metal``.
"""
from __future__ import annotations

from typing import Tuple

import torch


def gershgorin_is_psd(H: torch.Tensor, tol: float = 0.0) -> bool:
    """Sufficient (not necessary): diag - sum of off-diagonal magnitudes >= -tol for every row of a symmetric matrix."""
    d = torch.diagonal(H)
    off = H.abs().sum(-1) - d.abs()
    return bool(((d - off) >= -tol).all())


def min_eigenvalue(H: torch.Tensor) -> float:
    return float(torch.linalg.eigvalsh(H.double() if H.device.type == "cpu" else H.float())[0])


def project_psd(H: torch.Tensor, eps: float = 0.0) -> torch.Tensor:
    """Nearest (Frobenius) symmetric matrix with eigenvalues >= eps."""
    Hs = (H + H.transpose(-1, -2)) * 0.5
    w, V = torch.linalg.eigh(Hs.float())
    return ((V * w.clamp_min(eps).unsqueeze(-2)) @ V.transpose(-1, -2)).to(H.dtype)


def damp_until_cholesky(H: torch.Tensor, damp: float = 0.01, max_tries: int = 8) -> Tuple[torch.Tensor, torch.Tensor, float]:
    """(damped H, its lower Cholesky factor, damping used).  The damping starts at ``damp * mean(diag)`` and is multiplied
    by 10 after every failed factorization; the last resort is the PSD projection."""
    Hf = H.float()
    mean_diag = float(torch.diagonal(Hf).mean().clamp_min(1e-12))
    eye = torch.eye(H.shape[-1], device=H.device, dtype=torch.float32)
    lam = damp * mean_diag
    for _ in range(max_tries):
        Hd = Hf + lam * eye
        L, info = torch.linalg.cholesky_ex(Hd)
        if int(info) == 0:
            return Hd, L, lam
        lam *= 10.0
    Hd = project_psd(Hf, eps=damp * mean_diag)
    return Hd, torch.linalg.cholesky(Hd), float("nan")
