"""Hadamard transforms: fast Walsh-Hadamard on power-of-two blocks, block-diagonal rotation of weights and
activations, kurtosis (outlier) statistics.

Parity: reference ``metal_marlin/hadamard.py`` (``hadamard_matrix``, ``apply_hadamard_rotation``, block sizes
32-128, normalised so the transform is orthonormal and its own inverse) and the Metal ``hadamard.metal``
kernels.  On CUDA tensors ``block_hadamard`` runs the shared-memory butterfly kernel
(``csrc/misc_kernels.cu``); the PyTorch butterflies here are the CPU path and the oracle.
"""
from __future__ import annotations

import math

import torch


def hadamard_matrix(n: int, dtype=torch.float32, device=None) -> torch.Tensor:
    """Orthonormal Sylvester Hadamard matrix (``H @ H.T = I``); ``n`` a power of two."""
    if n & (n - 1) or n < 1:
        raise ValueError("Hadamard size must be a power of two")
    H = torch.ones(1, 1, dtype=torch.float64)
    while H.shape[0] < n:
        H = torch.cat([torch.cat([H, H], 1), torch.cat([H, -H], 1)], 0)
    return (H / math.sqrt(n)).to(dtype).to(device)


def fwht(x: torch.Tensor) -> torch.Tensor:
    """Orthonormal fast Walsh-Hadamard transform along the last axis (length a power of two)."""
    n = x.shape[-1]
    if n & (n - 1):
        raise ValueError("length must be a power of two")
    y = x.to(torch.float32).reshape(-1, n)
    h = 1
    while h < n:
        y = y.view(-1, n // (2 * h), 2, h)
        y = torch.stack([y[:, :, 0] + y[:, :, 1], y[:, :, 0] - y[:, :, 1]], 2).reshape(-1, n)
        h *= 2
    return (y / math.sqrt(n)).view(x.shape).to(x.dtype)


def block_hadamard(x: torch.Tensor, block: int = 128) -> torch.Tensor:
    """Apply the orthonormal Hadamard transform to consecutive ``block``-wide slices of the last axis (a
    block-diagonal rotation; it is its own inverse)."""
    D = x.shape[-1]
    if D % block:
        raise ValueError(f"last dimension {D} is not a multiple of the block {block}")
    if x.is_cuda:
        from .. import ops
        if ops.native_available() and x.dtype == torch.bfloat16 and block <= 1024:
            return ops.hadamard(x, block)
    return fwht(x.reshape(*x.shape[:-1], D // block, block)).reshape(x.shape)


def rotate_weight(w: torch.Tensor, block: int = 128) -> torch.Tensor:
    """``W' = W Hd`` for ``W [out, in]`` so that ``W' (Hd x) = W x`` (Hd symmetric, orthonormal)."""
    return block_hadamard(w.to(torch.float32), block).to(w.dtype)


def rotate_hessian(H: torch.Tensor, block: int = 128) -> torch.Tensor:
    """``Hd^T H Hd`` for the input-covariance Hessian of a rotated layer."""
    return block_hadamard(block_hadamard(H.to(torch.float32), block).t().contiguous(), block).t().contiguous()


def kurtosis(w: torch.Tensor, dim: int = -1) -> torch.Tensor:
    """Excess kurtosis along ``dim`` (0 for a Gaussian); heavy tails are what the rotation removes."""
    x = w.to(torch.float32)
    m = x.mean(dim, keepdim=True)
    c = x - m
    v = c.pow(2).mean(dim, keepdim=True).clamp_min(1e-30)
    return (c.pow(4).mean(dim, keepdim=True) / v.pow(2)).squeeze(dim) - 3.0
