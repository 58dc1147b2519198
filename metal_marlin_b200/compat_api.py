"""The reference facade's remaining public names on this engine: packing / unpacking helpers in the marlin ``[K, N]``
orientation, FP8 tables and KV helpers, Hadamard rotation with metadata, MoE dispatch bookkeeping, GEMM / attention entry
points with the reference's call signatures, RoPE / YaRN helpers, model-level quantization drivers, mask builders and
module-level generation functions.  Every function here is a thin layer over the kernels and modules of this package: the
names exist so that code written against ``metal_marlin`` finds them; nothing Metal-specific is emulated (``HAS_MPS`` is
False, the ``*_metal`` entry points run the CUDA kernels).

Parity: reference ``metal_marlin/__init__.py`` (``__all__``) with ``quantize.py`` (``pack_*_weights`` ``:112-940``,
``quantize_to_*``), ``fp8_utils.py`` (``:359``, ``:852``), ``hadamard.py`` (``:212``, ``:356``), ``moe_dispatch.py`` (``:453-952``),
``expert_ops.py`` (``:70``, ``:181``), ``attention.py`` (``:617-722``, ``:1180``), ``rope.py`` (``:133-512``), ``awq.py``,
``layer_replacement.py`` (``:237``, ``:258``), ``generate.py`` (``:163``, ``:228``).
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass, field
from typing import Any, Dict, Iterator, List, Optional, Sequence, Tuple

import numpy as np
import torch

from . import ops
from ._compat import E2M1_VALUES, NF4_VALUES
from .formats import fp4 as fp4fmt
from .quant import hadamard as _had
from .quant import rtn

HAS_MPS = False                 # no Metal Performance Shaders device on this platform
HAS_PYOBJC_METAL = False
HAS_CUDA_KERNELS = ops.native_available


def _to_torch(x) -> torch.Tensor:
    if isinstance(x, torch.Tensor):
        return x
    a = np.ascontiguousarray(np.asarray(x))
    if a.dtype == np.uint32:
        a = a.view(np.int32)                       # packed words: same bits, a dtype every torch op accepts
    return torch.from_numpy(a)


def _out(t: torch.Tensor, backend: str, dtype=None):
    if backend == "torch":
        return t if dtype is None else t.to(dtype)
    if backend == "numpy":
        a = t.detach().cpu().numpy()
        if a.dtype == np.int32 and dtype is None:
            a = a.view(np.uint32)                  # packed words are unsigned in the reference's arrays
        return a if dtype is None else a.astype(dtype)
    raise ValueError(f"output_backend {backend!r} is not available here (numpy | torch)")


# ------------------------------------------------------------------------------------------------ FP8 tables
def compute_fp8_e4m3_values() -> np.ndarray:
    """All 256 E4M3 (finite-only variant) code values, NaN codes as 0."""
    v = torch.arange(256, dtype=torch.uint8).view(torch.float8_e4m3fn).float()
    return torch.nan_to_num(v, nan=0.0).numpy()


def compute_fp8_e5m2_values() -> np.ndarray:
    v = torch.arange(256, dtype=torch.uint8).view(torch.float8_e5m2).float()
    return torch.nan_to_num(v, nan=0.0, posinf=57344.0, neginf=-57344.0).numpy()


FP8_E4M3_MAX, FP8_E5M2_MAX = 448.0, 57344.0
FP8_E4M3_VALUES, FP8_E5M2_VALUES = compute_fp8_e4m3_values(), compute_fp8_e5m2_values()


# ------------------------------------------------------------------------------------------------ packers, [K, N] orientation
def _pad_k(w: torch.Tensor, group_size: int, pad_k: bool) -> Tuple[torch.Tensor, Dict[str, int]]:
    K, N = w.shape
    mult = group_size if group_size % 8 == 0 else group_size * 8 // math.gcd(group_size, 8)
    Kp = -(-K // mult) * mult
    if Kp != K and not pad_k:
        raise ValueError(f"K={K} is not a multiple of group_size={group_size} (pass pad_k=True)")
    if Kp != K:
        w = torch.cat([w, torch.zeros(Kp - K, N, dtype=w.dtype)], 0)
    return w, {"orig_K": K, "orig_N": N, "padded_K": Kp, "padded_N": N, "group_size": group_size}


def _pack_generic(weights, group_size, pad_k, scales_dtype, output_backend, fmt: str, **kw):
    w, meta = _pad_k(_to_torch(weights).float(), group_size, pad_k)
    q = rtn.quantize(w.t().contiguous(), fmt, group_size) if not kw else rtn.QUANTIZERS[fmt](w.t().contiguous(), group_size, **kw)
    meta["format"] = fmt
    if q.bits == 4:
        packed = fp4fmt._pack_last_axis(q.codes).t().contiguous()          # [K / 8, N], eight codes along K per word
    else:
        packed = q.codes.t().contiguous()                                   # one byte per weight, [K, N]
    scales = q.scales.t().contiguous()
    out = (_out(packed, output_backend), _out(scales, output_backend, scales_dtype), meta)
    if q.zeros is not None:
        meta["zeros"] = _out(q.zeros.t().contiguous(), output_backend, scales_dtype)
    return out


def pack_fp4_weights(weights, group_size: int = 128, pad_k: bool = True, scales_dtype=None, output_backend: str = "numpy"):
    """``weights [K, N]`` -> ``(packed uint32-as-int32 [K_pad / 8, N], scales fp16 [K_pad / group_size, N], meta)``; E2M1 codes,
    ``scale = absmax / 6`` per group along K, K zero-padded to the group size."""
    return _pack_generic(weights, group_size, pad_k, scales_dtype, output_backend, "fp4")


def pack_fp4_weights_cpu(weights, group_size: int = 128, pad_k: bool = True, scales_dtype=None, output_backend: str = "numpy"):
    return pack_fp4_weights(_to_torch(weights).cpu(), group_size, pad_k, scales_dtype, output_backend)


def pack_int4_weights(weights, group_size: int = 128, pad_k: bool = True, scales_dtype=None, output_backend: str = "numpy"):
    """Symmetric INT4 (zero point 8) in the same layout; ``meta['zeros']`` holds the zero points."""
    return _pack_generic(weights, group_size, pad_k, scales_dtype, output_backend, "int4", symmetric=True)


def pack_nf4_weights(weights, group_size: int = 128, pad_k: bool = True, scales_dtype=None, output_backend: str = "numpy"):
    return _pack_generic(weights, group_size, pad_k, scales_dtype, output_backend, "nf4")


def pack_fp8_weights(weights, group_size: int = 128, format: str = "e4m3", pad_k: bool = True, scales_dtype=None,
                     output_backend: str = "numpy"):
    """One FP8 byte per weight ``[K_pad, N]`` + group scales."""
    w, meta = _pad_k(_to_torch(weights).float(), group_size, pad_k)
    q = rtn.quantize_fp8(w.t().contiguous(), group_size, variant=format)
    meta["format"] = "fp8_" + format
    return _out(q.codes.t().contiguous(), output_backend), _out(q.scales.t().contiguous(), output_backend, scales_dtype), meta


def _unpack_codes(packed: torch.Tensor, bits4: bool) -> torch.Tensor:
    """-> uint8 codes ``[N, K_pad]``."""
    p = _to_torch(packed)
    if bits4:
        return fp4fmt._unpack_last_axis(p.to(torch.int32).t().contiguous())
    return p.to(torch.uint8).t().contiguous()


def _dequant(packed, scales, meta, table, bits4=True, zeros=None) -> torch.Tensor:
    codes = _unpack_codes(packed, bits4).long()
    sc = _to_torch(scales).float().t()                                       # [N, groups]
    gs = meta["group_size"]
    vals = table.to(torch.float32)[codes] if table is not None else codes.float()
    vals = vals.view(codes.shape[0], -1, gs)
    if zeros is not None:
        vals = vals - _to_torch(zeros).float().t().unsqueeze(-1)
    w = (vals * sc.unsqueeze(-1)).view(codes.shape[0], -1).t()               # [K_pad, N]
    return w[: meta["orig_K"], : meta["orig_N"]].contiguous()


def unpack_fp4_weights(packed, scales, meta, weights_dtype=None, output_backend: str = "numpy"):
    """Inverse of :func:`pack_fp4_weights`: float ``[orig_K, orig_N]``."""
    w = _dequant(packed, scales, meta, torch.tensor(E2M1_VALUES))
    return _out(w, output_backend, weights_dtype or (np.float16 if output_backend == "numpy" else torch.float16))


def dequant_fp8_e4m3(packed, scales, meta, weights_dtype=None, output_backend: str = "numpy"):
    w = _dequant(packed, scales, meta, torch.from_numpy(FP8_E4M3_VALUES), bits4=False)
    return _out(w, output_backend, weights_dtype or (np.float16 if output_backend == "numpy" else torch.float16))


def dequant_fp8_e5m2(packed, scales, meta, weights_dtype=None, output_backend: str = "numpy"):
    w = _dequant(packed, scales, meta, torch.from_numpy(FP8_E5M2_VALUES), bits4=False)
    return _out(w, output_backend, weights_dtype or (np.float16 if output_backend == "numpy" else torch.float16))


def awq_dequantize(packed, scales, zeros, q_scale, meta, weights_dtype=None, output_backend: str = "numpy"):
    """INT4 codes with zero points, then the per-input-channel AWQ scale divided back out: ``w = (code - zero) * scale / q_scale``."""
    w = _dequant(packed, scales, meta, None, zeros=zeros)
    w = w / _to_torch(q_scale).float().view(-1, 1)[: w.shape[0]]
    return _out(w, output_backend, weights_dtype or (np.float16 if output_backend == "numpy" else torch.float16))


def dequantize_mmfp4(packed, scales, group_size: int = 128, dtype=torch.float32) -> torch.Tensor:
    """Row-packed MMFP4 ``[out, in / 8]`` + scales ``[out, groups]`` (or transposed) -> float ``[out, in]``."""
    codes, sc = fp4fmt.unpack_mmfp4(_to_torch(packed), _to_torch(scales))
    return fp4fmt.dequantize_codes(codes, sc, dtype)


# ------------------------------------------------------------------------------------------------ FP8 tensors and KV helpers
def _fp8_quant(x: torch.Tensor, dt, fmax: float, scale_method: str, group_size: int):
    xf = x.float()
    if scale_method == "tensor":
        s = (xf.abs().max() / fmax).clamp_min(1e-12).reshape(1)
        return (xf / s).to(dt).view(torch.uint8), s
    if scale_method == "channel":
        s = (xf.abs().amax(-1, keepdim=True) / fmax).clamp_min(1e-12)
        return (xf / s).to(dt).view(torch.uint8), s
    if scale_method == "group":
        g = xf.reshape(*xf.shape[:-1], -1, group_size)
        s = (g.abs().amax(-1, keepdim=True) / fmax).clamp_min(1e-12)
        return (g / s).to(dt).view(torch.uint8).reshape(xf.shape), s.squeeze(-1)
    raise ValueError(scale_method)


def _fp8_dequant(codes: torch.Tensor, scales: torch.Tensor, dt, output_dtype) -> torch.Tensor:
    v = codes.view(dt).float()
    if scales.numel() == 1 or scales.shape[-1] == 1:
        v = v * scales
    elif scales.shape == v.shape[:-1]:
        v = v * scales.unsqueeze(-1)
    else:                                                   # group scales [..., groups]
        g = v.shape[-1] // scales.shape[-1]
        v = (v.reshape(*v.shape[:-1], -1, g) * scales.unsqueeze(-1)).reshape(v.shape)
    return v.to(output_dtype or torch.bfloat16)


def quantize_to_fp8_e4m3(x, scale_method: str = "channel", group_size: int = 128):
    """Tensor -> ``(uint8 E4M3 codes, scales)``; scales per tensor, per row (last axis) or per group of the last axis."""
    return _fp8_quant(_to_torch(x), torch.float8_e4m3fn, FP8_E4M3_MAX, scale_method, group_size)


def quantize_to_fp8_e5m2(x, scale_method: str = "channel", group_size: int = 128):
    return _fp8_quant(_to_torch(x), torch.float8_e5m2, FP8_E5M2_MAX, scale_method, group_size)


def dequantize_fp8_e4m3(fp8_tensor, scales, output_dtype=None) -> torch.Tensor:
    return _fp8_dequant(_to_torch(fp8_tensor), _to_torch(scales), torch.float8_e4m3fn, output_dtype)


def dequantize_fp8_e5m2(fp8_tensor, scales, output_dtype=None) -> torch.Tensor:
    return _fp8_dequant(_to_torch(fp8_tensor), _to_torch(scales), torch.float8_e5m2, output_dtype)


def quantize_kv_cache_fp8(k, v, scale_method: str = "channel", group_size: int = 128):
    """``((k_codes, k_scales), (v_codes, v_scales))`` in E4M3."""
    return quantize_to_fp8_e4m3(k, scale_method, group_size), quantize_to_fp8_e4m3(v, scale_method, group_size)


def quantize_kv_cache_fp8_e5m2(k, v, scale_method: str = "channel", group_size: int = 128):
    return quantize_to_fp8_e5m2(k, scale_method, group_size), quantize_to_fp8_e5m2(v, scale_method, group_size)


def dequantize_kv_cache_fp8(k_fp8, k_scales, v_fp8, v_scales, output_dtype=None):
    return dequantize_fp8_e4m3(k_fp8, k_scales, output_dtype), dequantize_fp8_e4m3(v_fp8, v_scales, output_dtype)


def dequantize_kv_cache_fp8_e5m2(k_fp8, k_scales, v_fp8, v_scales, output_dtype=None):
    return dequantize_fp8_e5m2(k_fp8, k_scales, output_dtype), dequantize_fp8_e5m2(v_fp8, v_scales, output_dtype)


# ------------------------------------------------------------------------------------------------ FP4 / Hadamard objects
class FP4Metal:
    """E2M1 group quantizer object (``quantize`` / ``dequantize``); on a GPU the fused quantize + pack kernel does the work."""

    def quantize(self, values, group_size: int = 128):
        """``values [rows, cols]`` -> ``(codes uint8 [rows, cols], scales fp16 [rows, cols / group_size])``."""
        v = _to_torch(values)
        if v.is_cuda and v.dim() == 2 and ops.native_available():
            packed, scales = ops.fp4_quantize_pack(v.float() if v.dtype not in (torch.float32, torch.bfloat16) else v, group_size)
            return fp4fmt._unpack_last_axis(packed), scales
        return fp4fmt.quantize_codes(v.reshape(-1, v.shape[-1]), group_size)

    def dequantize(self, indices, scales, group_size: int = 128):
        return fp4fmt.dequantize_codes(_to_torch(indices), _to_torch(scales), torch.float32)


def quantize_fp4_metal(values, group_size: int = 128):
    return FP4Metal().quantize(values, group_size)


def dequantize_fp4_metal(indices, scales, group_size: int = 128):
    return FP4Metal().dequantize(indices, scales, group_size)


@dataclass
class HadamardMetadata:
    block_size: int
    orig_shape: Tuple[int, ...]
    padded_shape: Tuple[int, ...]
    axis: int = 0


def apply_hadamard_rotation(weights, block_size: int = 64, axis: int = 0):
    """Block-diagonal orthonormal Hadamard rotation along ``axis`` (zero-padded to the block size): ``(rotated, metadata)``."""
    w = _to_torch(weights).float()
    moved = w.movedim(axis, -1)
    n = moved.shape[-1]
    pad = (-n) % block_size
    if pad:
        moved = torch.cat([moved, torch.zeros(*moved.shape[:-1], pad)], -1)
    rot = _had.block_hadamard(moved.contiguous(), block_size).movedim(-1, axis)
    meta = HadamardMetadata(block_size, tuple(w.shape), tuple(rot.shape), axis)
    return (rot.numpy() if isinstance(weights, np.ndarray) else rot), meta


def inverse_hadamard_rotation(weights, metadata: HadamardMetadata):
    """The orthonormal block transform is its own inverse; padding is cut off again."""
    w = _to_torch(weights).float()
    back = _had.block_hadamard(w.movedim(metadata.axis, -1).contiguous(), metadata.block_size)
    back = back[..., : metadata.orig_shape[metadata.axis]].movedim(-1, metadata.axis).contiguous()
    return back.numpy() if isinstance(weights, np.ndarray) else back


def hadamard_transform_metal(x, block_size: int = 64, normalize: bool = True):
    """Walsh-Hadamard transform of consecutive ``block_size`` slices of the last axis (the Hadamard kernel on a GPU)."""
    t = _to_torch(x)
    y = ops.hadamard(t, block_size) if t.shape[-1] % block_size == 0 else apply_hadamard_rotation(t, block_size, axis=-1)[0]
    return y if normalize else y * math.sqrt(block_size)


class HadamardMetal:
    def transform(self, x, block_size: int = 64, normalize: bool = True):
        return hadamard_transform_metal(x, block_size, normalize)


# ------------------------------------------------------------------------------------------------ MoE dispatch bookkeeping
@dataclass
class MoEDispatchInfo:
    sorted_token_indices: torch.Tensor        # [T * k] token of every (token, slot) pair in expert order
    sorted_expert_indices: torch.Tensor       # [T * k] slot of every pair in expert order
    expert_offsets: torch.Tensor              # [E + 1]
    inverse_indices: torch.Tensor             # [T * k] position of pair (token * k + slot) in the sorted order
    num_tokens: int
    top_k: int
    num_experts: int


def group_tokens_by_expert(expert_ids: torch.Tensor, num_experts: int):
    """``expert_ids [T, k]`` -> ``(sorted_indices [T * k] into the flattened pairs, expert_offsets [E + 1], inverse_indices)``
    by a stable counting sort."""
    flat = expert_ids.reshape(-1).long()
    order = torch.sort(flat, stable=True).indices
    counts = torch.bincount(flat.clamp_min(0), minlength=num_experts)
    offsets = torch.zeros(num_experts + 1, dtype=torch.int64, device=flat.device)
    offsets[1:] = torch.cumsum(counts, 0)
    inverse = torch.empty_like(order)
    inverse[order] = torch.arange(order.numel(), device=order.device)
    return order, offsets, inverse


def group_tokens_by_expert_full(expert_ids: torch.Tensor, num_experts: int, use_gpu: bool = True) -> MoEDispatchInfo:
    T, k = expert_ids.shape
    order, offsets, inverse = group_tokens_by_expert(expert_ids, num_experts)
    return MoEDispatchInfo(order // k, order % k, offsets, inverse, T, k, num_experts)


def gather_for_experts(activations: torch.Tensor, dispatch_info: MoEDispatchInfo) -> torch.Tensor:
    return activations[dispatch_info.sorted_token_indices]


def scatter_expert_outputs(expert_outputs: torch.Tensor, expert_probs: torch.Tensor, dispatch_info: MoEDispatchInfo) -> torch.Tensor:
    """Expert-ordered rows back to tokens, weighted by ``expert_probs [T, k]`` and summed over the slots."""
    d = dispatch_info
    w = expert_probs[d.sorted_token_indices, d.sorted_expert_indices].to(expert_outputs.dtype).unsqueeze(-1)
    out = torch.zeros(d.num_tokens, expert_outputs.shape[-1], dtype=expert_outputs.dtype, device=expert_outputs.device)
    return out.index_add_(0, d.sorted_token_indices, expert_outputs * w)


def compute_expert_load(expert_ids: torch.Tensor, num_experts: int) -> torch.Tensor:
    return torch.bincount(expert_ids.reshape(-1).long(), minlength=num_experts)


def compute_load_balancing_loss(expert_probs_pre_topk: torch.Tensor, expert_ids: torch.Tensor, num_experts: int) -> torch.Tensor:
    from .moe.load_balancing import load_balance_loss
    return load_balance_loss(expert_probs_pre_topk, expert_ids, num_experts)


def expert_gather(expert_weights: torch.Tensor, expert_indices: torch.Tensor, output: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``expert_weights [E, ...]``, ``expert_indices [T, k]`` -> ``[T, k, ...]``."""
    g = expert_weights[expert_indices.long()]
    if output is not None:
        output.copy_(g)
        return output
    return g


def expert_scatter_add(expert_outputs: torch.Tensor, expert_indices: torch.Tensor, routing_weights: torch.Tensor,
                       output: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``expert_outputs [T, k, H]`` weighted by ``routing_weights [T, k]`` and summed over ``k`` -> ``[T, H]``."""
    y = (expert_outputs * routing_weights.to(expert_outputs.dtype).unsqueeze(-1)).sum(1)
    if output is not None:
        output.add_(y)
        return output
    return y


def fused_moe_forward(hidden: torch.Tensor, gate_up_packed: torch.Tensor, gate_up_scales: torch.Tensor, down_packed: torch.Tensor,
                      down_scales: torch.Tensor, expert_ids: torch.Tensor, probs: torch.Tensor) -> torch.Tensor:
    """Routed expert MLP from stacked row-packed MMFP4 tensors (``[E, out, in / 8]`` + scales ``[E, out, groups]`` or
    ``[E, groups, out]``) through this engine's expert kernels."""
    from .ops.weights import FP4ExpertBank, FP4Weight
    dev = hidden.device
    gu = FP4ExpertBank.from_weights([FP4Weight.from_mmfp4(gate_up_packed[e], gate_up_scales[e], dev) for e in range(gate_up_packed.shape[0])])
    dn = FP4ExpertBank.from_weights([FP4Weight.from_mmfp4(down_packed[e], down_scales[e], dev) for e in range(down_packed.shape[0])])
    x = hidden.reshape(-1, hidden.shape[-1]).to(torch.bfloat16)
    y = ops.moe_forward(x, gu, dn, expert_ids.reshape(x.shape[0], -1).to(torch.int32), probs.reshape(x.shape[0], -1).float())
    return y.reshape(*hidden.shape[:-1], -1)


class ExpertManagerCpp:
    """Token grouping through the native runtime (``csrc/runtime.cpp``) with the PyTorch sort as fallback."""

    def __init__(self, num_experts: int, top_k: int):
        self.num_experts, self.top_k = num_experts, top_k

    def group(self, expert_ids: torch.Tensor) -> MoEDispatchInfo:
        return group_tokens_by_expert_full(expert_ids, self.num_experts)

    def load_imbalance(self, expert_ids: torch.Tensor) -> float:
        load = compute_expert_load(expert_ids, self.num_experts).float()
        return float(load.max() / load.mean().clamp_min(1e-9))


def expert_manager_available() -> bool:
    return True


def create_expert_manager(num_experts: int, top_k: int) -> ExpertManagerCpp:
    return ExpertManagerCpp(num_experts, top_k)


# ------------------------------------------------------------------------------------------------ GEMM entry points
def marlin_gemm_fp4(A: torch.Tensor, B_packed: torch.Tensor, scales: torch.Tensor, group_size: int = 128) -> torch.Tensor:
    """``A [..., K] @ W [K, N]`` with ``B_packed [K / 8, N]`` / ``scales [K / group_size, N]`` (marlin layout).  The weight is
    brought into the device tile layout per call: keep a ``layers.MMFP4Linear`` for repeated use."""
    from .ops.weights import FP4Weight
    W = FP4Weight.from_marlin_fp4(B_packed.to(torch.int32), scales, A.device)
    x = A.reshape(-1, A.shape[-1]).to(torch.bfloat16)
    return ops.linear(x, W).reshape(*A.shape[:-1], -1)


def mmfp4_gemm(A: torch.Tensor, packed: torch.Tensor, scales: torch.Tensor, group_size: int = 128) -> torch.Tensor:
    """Same for the row-packed MMFP4 layout ``[out, in / 8]``."""
    from .ops.weights import FP4Weight
    W = FP4Weight.from_mmfp4(packed.to(torch.int32), scales, A.device)
    x = A.reshape(-1, A.shape[-1]).to(torch.bfloat16)
    return ops.linear(x, W).reshape(*A.shape[:-1], -1)


def marlin_gemm_int4(A: torch.Tensor, B_packed: torch.Tensor, scales: torch.Tensor, zeros: Optional[torch.Tensor] = None,
                     group_size: int = 128) -> torch.Tensor:
    """``B_packed [K / 8, N]`` unsigned INT4 codes, ``scales`` / ``zeros [K / group_size, N]`` (``zeros`` default 8)."""
    from .layers.linear import QuantizedLinear
    codes = fp4fmt._unpack_last_axis(B_packed.to(torch.int32).t().contiguous())
    z = zeros.t().contiguous() if zeros is not None else torch.full_like(scales.t(), 8.0).contiguous()
    lin = QuantizedLinear(rtn.QuantizedTensor(codes, scales.t().contiguous(), z, "int4", group_size, 4), None, A.device)
    return lin(A)


def mmfp4_fused_qkv(x: torch.Tensor, q: Tuple[torch.Tensor, torch.Tensor], k: Tuple[torch.Tensor, torch.Tensor],
                    v: Tuple[torch.Tensor, torch.Tensor]) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """One launch for the three projections: the row-packed ``(packed, scales)`` pairs are stacked along the output axis."""
    from .ops.weights import FP4Weight
    ws = [FP4Weight.from_mmfp4(p.to(torch.int32), s, x.device) for p, s in (q, k, v)]
    W = FP4Weight.concat_rows(ws)
    y = ops.linear(x.reshape(-1, x.shape[-1]).to(torch.bfloat16), W)
    a, b = ws[0].out_features, ws[0].out_features + ws[1].out_features
    lead = x.shape[:-1]
    return y[:, :a].reshape(*lead, -1), y[:, a:b].reshape(*lead, -1), y[:, b:].reshape(*lead, -1)


def dispatch_batched_gemm_variable_seq(lib, A: torch.Tensor, B: torch.Tensor, scales: torch.Tensor, N: int, K: int,
                                       batch_seq_lengths: Sequence[int], group_size: int = 128) -> torch.Tensor:
    """``A [sum(lengths), K]`` (sequences back to back) times one marlin-FP4 weight: ragged batches are just rows here
    (``lib`` is ignored; it named the Metal kernel library)."""
    assert A.shape[0] == int(sum(batch_seq_lengths)) and A.shape[1] == K
    return marlin_gemm_fp4(A, B, scales, group_size)[:, :N]


def dispatch_grouped_attention_variable_seq(lib, Q: torch.Tensor, K: torch.Tensor, scores: Optional[torch.Tensor],
                                            seq_lengths: torch.Tensor, max_seq_len: int, causal: bool = True,
                                            V: Optional[torch.Tensor] = None, scale: Optional[float] = None) -> torch.Tensor:
    """Variable-length attention over sequences stored back to back: ``Q [T, Hq, D]``, ``K`` (and ``V``) ``[T, Hk, D]``."""
    cu = torch.zeros(seq_lengths.numel() + 1, dtype=torch.int32, device=Q.device)
    cu[1:] = torch.cumsum(seq_lengths.to(torch.int32), 0)
    return ops.prefill_attention(Q, K, V if V is not None else K, cu, cu_k=cu, max_q=max_seq_len, scale=scale, causal=causal)


# ------------------------------------------------------------------------------------------------ attention entry points, masks
def _bhsd_attention(q, k, v, scale, causal, window=0):
    from .inference.prefill import flash_prefill_attention
    return flash_prefill_attention(q.to(torch.bfloat16), k.to(torch.bfloat16), v.to(torch.bfloat16), causal=causal, scale=scale,
                                   window=window).to(q.dtype)


def flash_attention_metal(q, k, v, scale: Optional[float] = None, causal: bool = True, num_kv_heads: Optional[int] = None):
    """``q [B, Hq, T, D]``, ``k, v [B, Hk, N, D]`` -> ``[B, Hq, T, D]`` on the prompt attention kernels."""
    return _bhsd_attention(q, k, v, scale, causal)


def sliding_window_attention_metal(q, k, v, window_size: int, scale: Optional[float] = None, causal: bool = True,
                                   num_kv_heads: Optional[int] = None):
    return _bhsd_attention(q, k, v, scale, causal, window=window_size)


def scaled_dot_product_attention_metal(q, k, v, attn_mask: Optional[torch.Tensor] = None, scale: Optional[float] = None,
                                       is_causal: bool = False):
    if attn_mask is None:
        return _bhsd_attention(q, k, v, scale, is_causal)
    return torch.nn.functional.scaled_dot_product_attention(q, k, v, attn_mask=attn_mask, scale=scale,
                                                            enable_gqa=q.shape[1] != k.shape[1])


def create_causal_mask(seq_len: int, kv_seq_len: Optional[int] = None, device=None) -> Optional[torch.Tensor]:
    """Additive mask ``[1, 1, seq_len, kv_seq_len]`` (0 visible, -inf hidden); queries are the last positions of the keys.
    ``None`` for a single query (nothing to hide)."""
    n = kv_seq_len or seq_len
    if seq_len == 1:
        return None
    qpos = torch.arange(n - seq_len, n, device=device).view(-1, 1)
    hidden = torch.arange(n, device=device).view(1, -1) > qpos
    return torch.zeros(seq_len, n, device=device).masked_fill(hidden, float("-inf")).view(1, 1, seq_len, n)


def create_sliding_window_mask(seq_len: int, window_size: int, kv_seq_len: Optional[int] = None, device=None) -> Optional[torch.Tensor]:
    n = kv_seq_len or seq_len
    qpos = torch.arange(n - seq_len, n, device=device).view(-1, 1)
    kpos = torch.arange(n, device=device).view(1, -1)
    hidden = (kpos > qpos) | (kpos <= qpos - window_size)
    return torch.zeros(seq_len, n, device=device).masked_fill(hidden, float("-inf")).view(1, 1, seq_len, n)


class MarlinAttention:
    """Multi-head attention block over FP4 projections: ``q / k / v / o`` are ``layers.MMFP4Linear``-like callables."""

    def __init__(self, q_proj, k_proj, v_proj, o_proj, num_heads: int, num_kv_heads: Optional[int] = None, rope=None,
                 window: int = 0):
        self.q_proj, self.k_proj, self.v_proj, self.o_proj = q_proj, k_proj, v_proj, o_proj
        self.num_heads, self.num_kv_heads, self.rope, self.window = num_heads, num_kv_heads or num_heads, rope, window

    def __call__(self, x: torch.Tensor, positions: Optional[torch.Tensor] = None) -> torch.Tensor:
        B, T, _ = x.shape
        q = self.q_proj(x).view(B, T, self.num_heads, -1)
        k = self.k_proj(x).view(B, T, self.num_kv_heads, -1)
        v = self.v_proj(x).view(B, T, self.num_kv_heads, -1)
        if self.rope is not None:
            pos = positions if positions is not None else torch.arange(T, device=x.device).expand(B, T)
            q, k = self.rope(q, pos), self.rope(k, pos)
        o = _bhsd_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), None, True, self.window)
        return self.o_proj(o.transpose(1, 2).reshape(B, T, -1))


# ------------------------------------------------------------------------------------------------ RoPE / YaRN
def get_yarn_mscale(scale_factor: float, mscale_all_dim: float = 0.0) -> float:
    if scale_factor <= 1.0:
        return 1.0
    m = mscale_all_dim if mscale_all_dim > 0 else 1.0
    return 0.1 * m * math.log(scale_factor) + 1.0


def compute_yarn_inv_freq(dim: int, base: float, config, device="cpu") -> torch.Tensor:
    from .rope import yarn_inv_freq
    import dataclasses
    cfg = dataclasses.replace(config, rope_theta=float(base)) if config.rope_theta != base else config
    return yarn_inv_freq(dim, cfg)[0].to(device)


def compute_yarn_cos_sin_cache(dim: int, max_seq_len: int, base: float, config, device="cpu", dtype=None):
    from .rope import cos_sin_cache, yarn_inv_freq
    import dataclasses
    cfg = dataclasses.replace(config, rope_theta=float(base)) if config.rope_theta != base else config
    inv, mscale = yarn_inv_freq(dim, cfg)
    cos, sin = cos_sin_cache(inv, max_seq_len, mscale, device)
    return (cos, sin) if dtype is None else (cos.to(dtype), sin.to(dtype))


class RoPE:
    """Rotary embedding callable: ``rope(x [B, T, H, D], positions [B, T])``."""

    def __init__(self, dim: int, base: float = 10000.0, scaling: Optional[dict] = None, interleaved: bool = False, max_position: int = 0):
        from .rope import rope_inv_freq
        self.dim, self.interleaved = dim, interleaved
        self.inv_freq, self.mscale = rope_inv_freq(dim, base, scaling, max_position or 4096)

    def __call__(self, x: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        from .rope import apply_rope
        B, T = x.shape[:2]
        y = apply_rope(x.reshape(B * T, *x.shape[2:]), positions.reshape(-1), self.inv_freq.to(x.device), interleaved=self.interleaved,
                       mscale=self.mscale)
        return y.reshape(x.shape)


class YaRNRoPE(RoPE):
    def __init__(self, dim: int, config, interleaved: bool = False):
        from .rope import yarn_inv_freq
        self.dim, self.interleaved, self.config = dim, interleaved, config
        self.inv_freq, self.mscale = yarn_inv_freq(dim, config)


def create_rope_from_config(config: Dict[str, Any], device="cpu") -> Optional[YaRNRoPE]:
    """A YaRN rotary embedding from a HF config dictionary; ``None`` when it configures no YaRN scaling."""
    from .rope import YaRNConfig
    yc = YaRNConfig.from_hf_config(config)
    if yc is None:
        return None
    dim = config.get("qk_rope_head_dim") or config.get("head_dim") or config["hidden_size"] // config["num_attention_heads"]
    return YaRNRoPE(dim, yc)


# ------------------------------------------------------------------------------------------------ AWQ statistics
def compute_activation_stats(activations, method: str = "rms") -> np.ndarray:
    """Per-input-channel importance of ``activations [..., in_features]``: mean |x|, max |x| or root mean square."""
    a = _to_torch(activations).float().reshape(-1, np.asarray(activations).shape[-1] if not isinstance(activations, torch.Tensor) else activations.shape[-1])
    s = {"mean": a.abs().mean(0), "max": a.abs().amax(0), "rms": a.pow(2).mean(0).sqrt()}[method]
    return s.numpy()


def find_salient_weights(weights, activation_stats, salient_ratio: float = 0.01):
    """``(mask over input channels, indices)`` of the ``salient_ratio`` share of channels with the largest statistics;
    ``weights [K, N]``."""
    st = _to_torch(activation_stats).float()
    n = max(1, int(round(st.numel() * salient_ratio)))
    idx = torch.topk(st, n).indices.sort().values
    mask = torch.zeros(st.numel(), dtype=torch.bool)
    mask[idx] = True
    return mask.numpy(), idx.numpy()


def compute_salient_scaling(weights, salient_mask, scales, group_size: int) -> np.ndarray:
    """Per-input-channel factor: salient channels are scaled up so that their largest weight reaches the largest weight of
    their quantization group (they then lose less to rounding); the others keep 1."""
    w = _to_torch(weights).float().abs()                       # [K, N]
    K = w.shape[0]
    grp_max = w.view(K // group_size, group_size, -1).amax((1, 2)).repeat_interleave(group_size)      # [K]
    row_max = w.amax(1).clamp_min(1e-12)
    s = torch.ones(K)
    m = _to_torch(salient_mask).bool()
    s[m] = (grp_max[m] / row_max[m]).clamp(1.0, 8.0)
    return s.numpy()


@dataclass
class AWQResult:
    packed: Any
    scales: Any
    zeros: Any
    q_scale: Any
    meta: Dict[str, Any] = field(default_factory=dict)


def awq_quantize_model(model_path, output_path, activations_path=None, group_size: int = 128, salient_ratio: float = 0.01,
                       activation_method: str = "rms", verbose: bool = True) -> Dict[str, Any]:
    """Whole-checkpoint AWQ through the offline pipeline (activation statistics are collected by a calibration pass of the
    model itself; ``activations_path`` is accepted for signature compatibility)."""
    from .quant.pipeline import quantize_checkpoint
    return quantize_checkpoint(str(model_path), str(output_path), fmt="mmfp4", method="awq", group_size=group_size)


# ------------------------------------------------------------------------------------------------ model-level quantization drivers
def _quantize_to(model_path, output_path, fmt: str, group_size: int, verbose: bool) -> Dict[str, Any]:
    from .quant.convert import convert_model
    info = convert_model(str(model_path), str(output_path), fmt, group_size)
    if verbose:
        print(f"quantized {info.get('quantized', '?')} tensors to {fmt} in {output_path}")
    return info


def quantize_to_fp8(model_path, output_path, group_size: int = 128, format: str = "e4m3", verbose: bool = True) -> Dict[str, Any]:
    return _quantize_to(model_path, output_path, "fp8", group_size, verbose)


def quantize_to_int4(model_path, output_path, group_size: int = 128, symmetric: bool = True, verbose: bool = True) -> Dict[str, Any]:
    return _quantize_to(model_path, output_path, "int4", group_size, verbose)


def quantize_to_nf4(model_path, output_path, group_size: int = 128, verbose: bool = True) -> Dict[str, Any]:
    return _quantize_to(model_path, output_path, "nf4", group_size, verbose)


def compute_hessian_metal(activations, normalize: bool = True) -> torch.Tensor:
    """``X^T X`` (divided by the row count when ``normalize``) in fp32 on the activations' device."""
    x = _to_torch(activations).float()
    x = x.reshape(-1, x.shape[-1])
    H = x.t() @ x
    return H / max(1, x.shape[0]) if normalize else H


def compute_moe_expert_sensitivity(expert_hessians: Sequence, router_logits=None) -> np.ndarray:
    """One score per expert: the trace of its Hessian (how much its inputs carry), weighted by how often the router picks
    it when logits are given; normalised to mean 1."""
    tr = torch.tensor([float(torch.as_tensor(np.asarray(h) if not isinstance(h, torch.Tensor) else h).float().diagonal().sum())
                       for h in expert_hessians], dtype=torch.float64)
    if router_logits is not None:
        p = torch.softmax(_to_torch(router_logits).double().reshape(-1, len(expert_hessians)), -1).mean(0)
        tr = tr * p * len(expert_hessians)
    return (tr / tr.mean().clamp_min(1e-30)).numpy()


class GPTQMetal:
    """Hessian + GPTQ object interface over ``quant.gptq`` (block kernel on a GPU)."""

    def compute_hessian(self, activations, normalize: bool = True) -> torch.Tensor:
        return compute_hessian_metal(activations, normalize)

    def quantize(self, weight: torch.Tensor, hessian: torch.Tensor, fmt: str = "fp4", group_size: int = 128, act_order: bool = False):
        from .quant.gptq import GPTQConfig, gptq_quantize
        return gptq_quantize(weight, hessian, GPTQConfig(fmt=fmt, group_size=group_size, act_order=act_order))


class GPTQQuantizer:
    """``quantize_weight(w [out, in], H) -> (w_q, scales, stats)`` with the configuration given at construction."""

    def __init__(self, bits: int = 4, group_size: int = 128, damp: float = 0.01, act_order: bool = False, fmt: Optional[str] = None):
        from .quant.gptq import GPTQConfig
        self.cfg = GPTQConfig(fmt=fmt or {8: "int8", 4: "int4", 3: "int3", 2: "int2"}[bits], group_size=group_size, damp=damp,
                              act_order=act_order)

    def quantize_weight(self, w: torch.Tensor, H: torch.Tensor):
        from .quant.gptq import gptq_quantize
        return gptq_quantize(w, H, self.cfg)


class FP4GPTQQuantizer(GPTQQuantizer):
    def __init__(self, group_size: int = 128, damp: float = 0.01, act_order: bool = False):
        super().__init__(4, group_size, damp, act_order, fmt="fp4")


class MRGPTQQuantizer:
    """Block-Hadamard rotation (kurtosis gated) + GPTQ."""

    def __init__(self, group_size: int = 128, hadamard_block: int = 128, fmt: str = "fp4", **kw):
        from .quant.gptq import MRGPTQConfig
        self.cfg = MRGPTQConfig(fmt=fmt, group_size=group_size, hadamard_block=hadamard_block, **kw)

    def quantize_weight(self, w: torch.Tensor, H: Optional[torch.Tensor] = None):
        from .quant.gptq import mr_gptq_quantize
        return mr_gptq_quantize(w, H, self.cfg)


class HessianManager:
    """Named Hessian accumulation (``add`` / ``get`` / ``save`` / ``load``): the calibration collector under its reference name."""

    def __new__(cls, *a, **k):
        from .quant.calibration import HessianCollector
        return HessianCollector(*a, **k)


# ------------------------------------------------------------------------------------------------ module replacement helpers
def get_parent_module(model, name: str):
    """``("model.layers.0.mlp") -> (module model.layers.0, "mlp")``."""
    parts = name.split(".")
    parent = model
    for p in parts[:-1]:
        parent = parent[int(p)] if p.isdigit() and hasattr(parent, "__getitem__") else getattr(parent, p)
    return parent, parts[-1]


def quantize_linear_layer(linear, bits: int = 4, group_size: int = 128, format: str = "fp4"):
    """``nn.Linear`` -> the quantized ``nn.Module`` that ``hf.replace_linear_layers`` installs."""
    from .hf import QuantizedLinearModule
    from .layers.linear import MMFP4Linear, QuantizedLinear
    w, dev = linear.weight.data, linear.weight.device
    fmt = format if format not in ("int", "uint") else f"int{bits}"
    bias = None if linear.bias is None else linear.bias.data
    inner = (MMFP4Linear.from_float(w.float(), group_size, bias=None if bias is None else bias.to(dev, torch.bfloat16), device=dev)
             if fmt == "fp4" else QuantizedLinear.from_float(w.float(), fmt, group_size, bias=bias, device=dev))
    return QuantizedLinearModule(inner, linear.in_features, linear.out_features)


# ------------------------------------------------------------------------------------------------ module-level generation
def generate_stream(model, input_ids, config=None) -> Iterator[int]:
    """Yield the new token ids of one sequence as they are produced; ``model``: ``MMFP4ForCausalLM``; ``config``: an
    object with ``max_new_tokens`` / ``temperature`` / ``top_k`` / ``top_p`` / ``eos_token_id`` (all optional)."""
    ids = [int(t) for t in (input_ids.reshape(-1).tolist() if isinstance(input_ids, torch.Tensor) else input_ids)]
    n = int(getattr(config, "max_new_tokens", 64))
    eos = getattr(config, "eos_token_id", None)
    eos = set(eos if isinstance(eos, (list, tuple, set)) else [eos]) - {None}
    from .sampler import SamplingConfig, sample_next_token
    temp = float(getattr(config, "temperature", 0.0))
    sc = SamplingConfig(temperature=temp, top_k=int(getattr(config, "top_k", 0)), top_p=float(getattr(config, "top_p", 1.0)),
                        do_sample=temp > 0)
    generated: List[int] = []
    if temp == 0.0 and n > 0:
        # greedy: the persistent decode state (paged cache, one captured step per token) instead of re-running the prompt
        from .inference.decode import DecodeConfig, DecodeState, persistent_decode_step
        st = DecodeState(model, DecodeConfig(batch_size=1, max_context=len(ids) + n + 16, max_new_tokens=n + 1))
        tok = int(st.prefill([ids])[0])
        for i in range(n):
            yield tok
            if tok in eos or i + 1 == n:
                return
            tok = int(persistent_decode_step(st)[0])
        return
    for _ in range(n):
        logits = model.forward_logits(ids)                      # [tokens, vocab]: the last row predicts the next token
        tok = int(sample_next_token(logits.reshape(len(ids), -1)[-1].reshape(1, -1), sc, generated))
        generated.append(tok)
        ids.append(tok)
        yield tok
        if tok in eos:
            return


def generate(model, input_ids, config=None) -> List[int]:
    return list(generate_stream(model, input_ids, config))


def generate_batch(model, input_ids, config=None, attention_mask=None) -> List[List[int]]:
    """New tokens of every row of ``input_ids [B, T]`` (rows right-padded rows are cut by ``attention_mask``), greedy or
    sampled by the engine's batched decode."""
    rows = input_ids.tolist() if isinstance(input_ids, torch.Tensor) else [list(r) for r in input_ids]
    if attention_mask is not None:
        rows = [[t for t, m in zip(r, mr) if m] for r, mr in zip(rows, attention_mask.tolist())]
    return model.generate(rows, max_new_tokens=int(getattr(config, "max_new_tokens", 64)))


# ------------------------------------------------------------------------------------------------ precision configuration
import enum as _enum


class Precision(_enum.Enum):
    FP16 = "fp16"
    BF16 = "bf16"
    FP8 = "fp8"
    INT8 = "int8"
    FP4 = "fp4"
    INT4 = "int4"
    NF4 = "nf4"
    INT3 = "int3"
    INT2 = "int2"

    @property
    def bits(self) -> int:
        return {"fp16": 16, "bf16": 16, "fp8": 8, "int8": 8, "fp4": 4, "int4": 4, "nf4": 4, "int3": 3, "int2": 2}[self.value]


QuantizationFormat = Precision


@dataclass
class LayerQuantConfig:
    name: str
    precision: Precision
    group_size: int = 128

    @property
    def quantized(self) -> bool:
        return self.precision.bits < 16


@dataclass
class MoEPrecisionConfig:
    router: Precision = Precision.BF16
    experts: Precision = Precision.FP4
    shared_expert: Precision = Precision.FP4
    expert_group_size: int = 128


@dataclass
class MixedPrecisionConfig:
    """Precision per tensor class; ``from_preset`` gives the named presets (dense / moe / moe-mtp / quality / speed)."""
    default: Precision = Precision.FP4
    attention: Precision = Precision.FP4
    mlp: Precision = Precision.FP4
    embeddings: Precision = Precision.BF16
    lm_head: Precision = Precision.BF16
    norms: Precision = Precision.BF16
    group_size: int = 128
    moe: MoEPrecisionConfig = field(default_factory=MoEPrecisionConfig)
    preset: str = "dense"

    @classmethod
    def from_preset(cls, name: str) -> "MixedPrecisionConfig":
        from .quant.mixed_precision import policy_for

        def prec(tensor: str) -> Precision:
            p = policy_for(tensor, name)
            fmt = getattr(p, "fmt", None) or getattr(p, "format", None)
            return Precision(fmt) if fmt in Precision._value2member_map_ else Precision.BF16
        gs = getattr(policy_for("model.layers.0.mlp.down_proj.weight", name), "group_size", 128) or 128
        return cls(default=prec("model.layers.0.mlp.down_proj.weight"), attention=prec("model.layers.0.self_attn.q_proj.weight"),
                   mlp=prec("model.layers.0.mlp.down_proj.weight"), group_size=gs, preset=name,
                   moe=MoEPrecisionConfig(experts=prec("model.layers.1.mlp.experts.0.down_proj.weight"),
                                          shared_expert=prec("model.layers.1.mlp.shared_experts.down_proj.weight")))


class LayerPrecisionSelector:
    """``select(tensor name) -> LayerQuantConfig`` by tensor class under a :class:`MixedPrecisionConfig`."""

    def __init__(self, config: Optional[MixedPrecisionConfig] = None):
        self.config = config or MixedPrecisionConfig()

    def select(self, name: str) -> LayerQuantConfig:
        c = self.config
        if "norm" in name:
            return LayerQuantConfig(name, c.norms, c.group_size)
        if "embed_tokens" in name:
            return LayerQuantConfig(name, c.embeddings, c.group_size)
        if "lm_head" in name:
            return LayerQuantConfig(name, c.lm_head, c.group_size)
        if "mlp.gate.weight" in name or ".router." in name:
            return LayerQuantConfig(name, c.moe.router, c.group_size)
        if "shared_expert" in name:
            return LayerQuantConfig(name, c.moe.shared_expert, c.moe.expert_group_size)
        if ".experts." in name:
            return LayerQuantConfig(name, c.moe.experts, c.moe.expert_group_size)
        if "self_attn" in name or "attention" in name:
            return LayerQuantConfig(name, c.attention, c.group_size)
        if "mlp" in name:
            return LayerQuantConfig(name, c.mlp, c.group_size)
        return LayerQuantConfig(name, c.default, c.group_size)


@dataclass
class LayerSensitivity:
    name: str
    num_params: int
    error_by_bits: Dict[int, float]          # quantization error (any consistent metric) at each candidate bit width


@dataclass
class LayerBudget:
    name: str
    bits: int
    nbytes: int


@dataclass
class ModelBudgetAllocation:
    layers: List[LayerBudget]
    mean_bpw: float
    total_bytes: int

    def bits_for(self, name: str) -> int:
        return next(l.bits for l in self.layers if l.name == name)


@dataclass
class AdaptiveQuantResult:
    allocation: ModelBudgetAllocation
    target_bpw: float
    estimated_error: float


class AdaptiveQuantizer:
    """Sensitivity-driven bit allocation: the greedy marginal-gain search of ``quant.mixed_precision.allocate_bits`` behind
    the reference's object interface."""

    def __init__(self, target_bpw: float = 4.0, bit_choices: Sequence[int] = (2, 3, 4, 5, 6, 8)):
        self.target_bpw, self.bit_choices = target_bpw, tuple(bit_choices)

    def allocate(self, sensitivities: Sequence[LayerSensitivity]) -> AdaptiveQuantResult:
        from .quant.mixed_precision import allocate_bits
        sens = {s.name: dict(s.error_by_bits) for s in sensitivities}
        sizes = {s.name: s.num_params for s in sensitivities}
        bits = allocate_bits(sens, sizes, self.target_bpw, self.bit_choices)
        layers = [LayerBudget(n, int(b), sizes[n] * int(b) // 8) for n, b in bits.items()]
        total = sum(l.nbytes for l in layers)
        n_par = max(1, sum(sizes.values()))
        err = sum(sens[n].get(int(b), 0.0) for n, b in bits.items())
        return AdaptiveQuantResult(ModelBudgetAllocation(layers, total * 8 / n_par, total), self.target_bpw, err)


@dataclass
class QuantizationReport:
    """Per-tensor outcome of a quantization run (name, format, bits, relative error) with totals and JSON export."""
    entries: List[Dict[str, Any]] = field(default_factory=list)

    def add(self, name: str, fmt: str, bits: int, rel_error: float, num_params: int) -> None:
        self.entries.append({"name": name, "format": fmt, "bits": bits, "rel_error": rel_error, "num_params": num_params})

    def summary(self) -> Dict[str, Any]:
        n = sum(e["num_params"] for e in self.entries) or 1
        return {"tensors": len(self.entries), "mean_bpw": sum(e["bits"] * e["num_params"] for e in self.entries) / n,
                "mean_rel_error": sum(e["rel_error"] * e["num_params"] for e in self.entries) / n,
                "worst": max(self.entries, key=lambda e: e["rel_error"])["name"] if self.entries else None}

    def to_json(self) -> str:
        import json
        return json.dumps({"summary": self.summary(), "entries": self.entries})


# ------------------------------------------------------------------------------------------------ layers and modules under reference names
def __getattr__(name: str):
    lazy = {"MarlinLinear": (".layers.linear", "MMFP4Linear"), "MetalQuantizedLinear": (".hf", "QuantizedLinearModule"),
            "MetalQuantizedMoE": (".hf", "QuantizedMoEBlock"), "LLaVAProjector": (".vision", "LlavaProjector"),
            "Qwen2VLProjector": (".vision", "PatchMergerProjector"), "InternVLProjector": (".vision", "PixelShuffleProjector"),
            "CacheConfigTorch": (".kv.contiguous", "CacheConfig"), "MetalHeapAllocator": (".memory.arena", "Arena"),
            "HeapBufferPool": (".memory.pools", "BufferPool"), "HeapAllocatorMetrics": (".memory.pools", "BufferPoolStats")}
    if name in lazy:
        import importlib
        mod, attr = lazy[name]
        return getattr(importlib.import_module(mod, __package__), attr)
    raise AttributeError(name)


@dataclass
class VisionProjectorConfig:
    projector_type: str = "llava"          # llava | qwen2_vl | internvl | perceiver
    vision_hidden_size: int = 1024
    text_hidden_size: int = 4096
    merge_size: int = 2
    downsample_ratio: float = 0.5


def detect_projector_type(config: Dict[str, Any]) -> str:
    """``llava`` / ``qwen2_vl`` / ``internvl`` from a HF config dictionary (model type, then characteristic keys)."""
    mt = str(config.get("model_type", "")).lower()
    if "qwen2_vl" in mt or "qwen2_5_vl" in mt or "spatial_merge_size" in str(config.get("vision_config", {})):
        return "qwen2_vl"
    if "internvl" in mt or "downsample_ratio" in config:
        return "internvl"
    return "llava"


class VisionProjector:
    """Builds the projector of a family from its weights: ``VisionProjector.build(config, weights)`` with ``weights`` a
    dictionary ``{"w1", "b1", "w2", "b2"[, "ln_w", "ln_b"]}``."""

    @staticmethod
    def build(config: VisionProjectorConfig, weights: Dict[str, torch.Tensor]):
        from . import vision
        w = weights
        if config.projector_type == "llava":
            return vision.LlavaProjector(w["w1"], w.get("b1"), w["w2"], w.get("b2"))
        if config.projector_type == "qwen2_vl":
            return vision.PatchMergerProjector(w["ln_w"], w["ln_b"], w["w1"], w.get("b1"), w["w2"], w.get("b2"), config.merge_size)
        if config.projector_type == "internvl":
            return vision.PixelShuffleProjector(w["ln_w"], w["ln_b"], w["w1"], w.get("b1"), w["w2"], w.get("b2"), config.downsample_ratio)
        raise ValueError(config.projector_type)


# ------------------------------------------------------------------------------------------------ ONNX helpers
@dataclass
class ONNXGraphInfo:
    ops: List[Any]
    inputs: List[str]
    outputs: List[str]
    initializers: Dict[str, Tuple[Tuple[int, ...], str]]
    op_counts: Dict[str, int]
    architecture: str
    num_layers: int


def parse_onnx_graph_full(onnx_path) -> ONNXGraphInfo:
    from .converters import onnx as ox
    g = ox.load_onnx(onnx_path)
    inits = {k: (tuple(v.shape), str(v.dtype)) for k, v in g.initializers.items()}
    return ONNXGraphInfo(g.nodes, list(g.inputs), list(g.outputs), inits, ox._count_op_types(g.nodes), ox.detect_architecture(g.nodes),
                         ox.get_layer_count(g.nodes))


def list_onnx_tensors(onnx_path) -> List[Dict[str, Any]]:
    from .converters import onnx as ox
    g = ox.load_onnx(onnx_path)
    return [{"name": k, "shape": list(v.shape), "dtype": str(v.dtype), "size_bytes": int(v.nbytes)} for k, v in g.initializers.items()]


def normalize_onnx_name(onnx_name: str, consumer_map: Optional[Dict[str, List[str]]] = None) -> str:
    """ONNX path-style names (``/model/layers.0/self_attn/q_proj/MatMul``, ``onnx::MatMul_123`` resolved through the node
    that consumes it) -> HF tensor names (``model.layers.0.self_attn.q_proj.weight``)."""
    name = onnx_name
    if name.startswith("onnx::") and consumer_map and consumer_map.get(name):
        name = consumer_map[name][0]
    name = name.strip("/").replace("/", ".")
    for op in (".MatMul", ".Gemm", ".Add", ".Mul", ".Gather"):
        if name.endswith(op):
            name = name[: -len(op)]
    if not name.endswith((".weight", ".bias")):
        name += ".weight"
    return name


def extract_onnx_weights(onnx_path) -> Iterator[Tuple[str, np.ndarray, Dict[str, Any]]]:
    """``(HF-style name, array, metadata)`` for every initializer; MatMul weights are transposed to ``[out, in]``."""
    from .converters import onnx as ox
    g = ox.load_onnx(onnx_path)
    consumers: Dict[str, List[str]] = {}
    kinds: Dict[str, str] = {}
    for op in g.nodes:
        for i in op.inputs:
            consumers.setdefault(i, []).append(op.name or op.op_type)
            kinds.setdefault(i, op.op_type)
    for k, v in g.initializers.items():
        arr = np.asarray(v)
        transposed = kinds.get(k) == "MatMul" and arr.ndim == 2
        yield normalize_onnx_name(k, consumers), (arr.T.copy() if transposed else arr), {"onnx_name": k, "transposed": transposed,
                                                                                         "consumer": kinds.get(k)}


def get_onnx_config(onnx_path):
    """A ``ModelConfig`` inferred from tensor shapes (hidden size, layers, vocabulary, MLP width) of an exported decoder."""
    from .converters import onnx as ox
    from .models.config import ModelConfig
    g = ox.load_onnx(onnx_path)
    two_d = [np.asarray(v).shape for v in g.initializers.values() if np.asarray(v).ndim == 2]
    if not two_d:
        raise ValueError("no 2-D initializers: not a decoder export")
    dims = [d for s in two_d for d in s]
    hidden = max(set(dims), key=dims.count)
    other = sorted({d for s in two_d for d in s if d != hidden})
    vocab = max(other) if other and max(other) > 8 * hidden else 0
    inter = max((d for d in other if d != vocab), default=4 * hidden)
    layers = max(1, ox.get_layer_count(g.nodes))
    heads = max(1, hidden // 128) if hidden % 128 == 0 else max(1, hidden // 64)
    return ModelConfig(model_type=ox.detect_architecture(g.nodes) or "llama", vocab_size=vocab or 32000, hidden_size=hidden,
                       num_hidden_layers=layers, num_attention_heads=heads, num_key_value_heads=heads, head_dim=hidden // heads,
                       intermediate_size=inter)


# ------------------------------------------------------------------------------------------------ memory and dispatch objects
@dataclass
class HeapAllocation:
    offset: int
    size: int
    tensor: Optional[torch.Tensor] = None


@dataclass
class AsyncTransferHandle:
    tensors: Dict[str, torch.Tensor]
    event: Any = None

    def wait(self) -> Dict[str, torch.Tensor]:
        if self.event is not None:
            self.event.synchronize()
        return self.tensors

    def done(self) -> bool:
        return self.event is None or bool(self.event.query())


class AsyncTransferManager:
    """Host -> device transfers on a side stream through pinned staging (``memory.TransferStream``) with handles."""

    def __init__(self, device="cuda:0"):
        from .memory.pools import TransferStream
        self._ts = TransferStream(device if torch.cuda.is_available() else "cpu")

    def submit(self, tensors: Dict[str, torch.Tensor]) -> AsyncTransferHandle:
        out, ev = self._ts.transfer_async(tensors)
        return AsyncTransferHandle(out, ev)

    def synchronize(self) -> None:
        self._ts.synchronize()


def fast_dispatch_available() -> bool:
    """True when the native extension (kernels + launch glue) is loaded."""
    return bool(ops.native_available())


def mla_cpp_available() -> bool:
    return bool(ops.native_available())


class FastInferenceContext:
    """Process-wide handle on the native side: device, launch counter, status word."""

    def __init__(self, device=None):
        self.device = torch.device(device or ("cuda" if torch.cuda.is_available() else "cpu"))

    @property
    def available(self) -> bool:
        return fast_dispatch_available() and self.device.type == "cuda"

    def launch_count(self) -> int:
        return int(ops.launch_count())

    def check_status(self) -> int:
        return int(ops.check_status(self.device)) if self.available else 0


_fast_ctx: Optional[FastInferenceContext] = None


def get_fast_context() -> FastInferenceContext:
    global _fast_ctx
    if _fast_ctx is None:
        _fast_ctx = FastInferenceContext()
    return _fast_ctx


class BatchDispatchContext:
    """Queue many kernel launches and commit them as one: inside the ``with`` block the launches are captured into a CUDA
    graph (after the block's body ran once eagerly for warm-up when ``warmup``), ``commit()`` / leaving the block replays
    it.  On a CPU the body simply runs.  Use with a closure: ``with BatchDispatchContext() as b: b.run(fn)``."""

    def __init__(self, device=None, warmup: bool = True):
        self.device = torch.device(device or ("cuda" if torch.cuda.is_available() else "cpu"))
        self.warmup, self.graph, self._fn = warmup, None, None

    def __enter__(self):
        return self

    def run(self, fn) -> None:
        self._fn = fn
        if self.device.type != "cuda":
            fn()
            return
        if self.warmup:
            s = torch.cuda.Stream(self.device)
            s.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(s):
                fn()
            torch.cuda.current_stream(self.device).wait_stream(s)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            fn()

    def commit(self) -> None:
        if self.graph is not None:
            self.graph.replay()
        elif self._fn is not None and self.device.type != "cuda":
            self._fn()

    def __exit__(self, *exc):
        if exc[0] is None and self.graph is not None:
            self.graph.replay()
        return False


@dataclass
class CppDispatchInfo:
    """Device-built MoE work list: token order, its inverse, and per tile (expert, first row, rows)."""
    order: torch.Tensor
    inverse: torch.Tensor
    tile_expert: torch.Tensor
    tile_row0: torch.Tensor
    tile_rows: torch.Tensor
    num_tiles: torch.Tensor

    @classmethod
    def build(cls, expert_ids: torch.Tensor, num_experts: int, token_tile: int = 32) -> "CppDispatchInfo":
        order, te, r0, rw, nt = ops._build_tile_list(expert_ids.reshape(-1).long(), num_experts, token_tile)
        inverse = torch.empty_like(order)
        inverse[order.long()] = torch.arange(order.numel(), device=order.device, dtype=order.dtype)
        return cls(order, inverse, te, r0, rw, nt)


class PipelinedLayerDispatcher:
    """Runs ``layer_fn(i, weights)`` over layers whose weights live on the host while the next layers' weights are already
    on their way to the device (``memory.WeightStreamer``, ``depth`` layers ahead)."""

    def __init__(self, device=None, depth: int = 2):
        from .memory.streaming import WeightStreamer
        self.streamer = WeightStreamer(device or ("cuda" if torch.cuda.is_available() else "cpu"), depth)

    def run(self, host_layers: Sequence[Dict[str, torch.Tensor]], layer_fn, x):
        for i, w in enumerate(self.streamer.stream_layers(host_layers)):
            x = layer_fn(i, w, x)
        return x


class MLAAttentionCpp:
    """Absorbed MLA decode over the paged latent cache through the native launchers: ``decode(q_lat [B, H, R + dr],
    latent_pool, block_tables, ctx_lens, scale)`` returns the latent-space output ``[B, H, R]``."""

    def __init__(self, num_heads: int, kv_lora_rank: int, rope_dim: int, block_size: int = 16):
        self.H, self.R, self.dr, self.block_size = num_heads, kv_lora_rank, rope_dim, block_size

    @staticmethod
    def available() -> bool:
        return mla_cpp_available()

    def decode(self, q_lat: torch.Tensor, latent_pool, block_tables: torch.Tensor, ctx_lens: torch.Tensor, scale: float) -> torch.Tensor:
        return ops.paged_attention(q_lat, latent_pool, None, block_tables, ctx_lens, Hq=self.H, Hkv=1, dqk=self.R + self.dr, dv=self.R,
                                   block_size=self.block_size, scale=scale)


# ------------------------------------------------------------------------------------------------ GEMM operation objects
class GemmFp4:
    """``forward(x [..., K], packed_weight [K / 8, N], scales [K / group, N]) -> [..., N]`` on the FP4 GEMM / GEMV kernels
    (reference ``ops/gemm_fp4.py:20``).  Device weights are cached per packed tensor, so repeated calls with the same weight do
    not rebuild the tile layout."""

    def __init__(self, library: Any = None, cache_size: int = 64):
        self._cache: Dict[Tuple[int, int], Any] = {}
        self._cache_size = cache_size

    def _weight(self, packed: torch.Tensor, scales: torch.Tensor, device):
        from .ops.weights import FP4Weight
        key = (packed.data_ptr(), scales.data_ptr())
        hit = self._cache.get(key)
        if hit is not None and hit[0] is packed:
            return hit[1]
        W = FP4Weight.from_marlin_fp4(packed.to(torch.int32), scales, device)
        if len(self._cache) >= self._cache_size:
            self._cache.pop(next(iter(self._cache)))
        self._cache[key] = (packed, W)
        return W

    def forward(self, x: torch.Tensor, packed_weight: torch.Tensor, scales: torch.Tensor, group_size: int = 128) -> torch.Tensor:
        W = self._weight(packed_weight, scales, x.device)
        y = ops.linear(x.reshape(-1, x.shape[-1]).to(torch.bfloat16), W)
        return y.to(x.dtype if x.is_floating_point() else torch.bfloat16).reshape(*x.shape[:-1], -1)

    __call__ = forward


def pack_int8_weights(weights: torch.Tensor) -> torch.Tensor:
    """``[K, N]`` weights in ``[-1, 1]`` -> int8 codes ``round(w * 127)`` packed four to a word along K: ``[ceil(K / 4), N]`` (int32
    holding the uint32 bit pattern; byte ``i`` of a word is row ``4 r + i``).  Reference ``ops/gemm_int8.py:165``."""
    q = torch.clamp(torch.round(weights.float() * 127.0), -128, 127).to(torch.int32)
    K, N = q.shape
    pad = (-K) % 4
    if pad:
        q = torch.cat([q, torch.zeros(pad, N, dtype=torch.int32, device=q.device)])
    b = (q & 0xFF).view(-1, 4, N).to(torch.int64)
    word = b[:, 0] | (b[:, 1] << 8) | (b[:, 2] << 16) | (b[:, 3] << 24)
    return torch.where(word >= 2 ** 31, word - 2 ** 32, word).to(torch.int32)


def unpack_int8_weights(packed: torch.Tensor, K: Optional[int] = None) -> torch.Tensor:
    """Inverse of :func:`pack_int8_weights`: signed int8 values ``[K, N]``."""
    w = packed.to(torch.int64) & 0xFFFFFFFF
    b = torch.stack([(w >> s) & 0xFF for s in (0, 8, 16, 24)], 1).reshape(-1, packed.shape[-1])
    q = torch.where(b >= 128, b - 256, b).to(torch.int8)
    return q[:K] if K is not None else q


class GemmInt8:
    """W8A16: ``forward(activations [M, K], weights [K / 4, N] packed int8, scales [K / group, N], zeros) -> [M, N]`` with
    ``w = (q - zero) * scale`` (reference ``ops/gemm_int8.py:35``), on the code-table GEMM / GEMV kernels."""

    def __init__(self, device: Optional[str] = None):
        self.device = device
        self._cache: Dict[int, Any] = {}

    def _linear(self, weights, scales, zeros, group_size: int, K: int, device):
        hit = self._cache.get(weights.data_ptr())
        if hit is not None and hit[0] is weights:
            return hit[1]
        from .layers import QuantizedLinear
        from .quant.rtn import QuantizedTensor
        q = unpack_int8_weights(weights, K)                                   # [K, N]
        codes = (q.to(torch.int16) + 128).to(torch.uint8).t().contiguous()    # [N, K]
        z = torch.zeros_like(scales) if zeros is None else zeros
        qt = QuantizedTensor(codes, scales.t().contiguous().to(torch.float16), (z.t().contiguous().float() + 128.0).to(torch.float16), "int8",
                             group_size, 8)
        lin = QuantizedLinear(qt, None, device)
        self._cache = {weights.data_ptr(): (weights, lin)} if len(self._cache) > 32 else {**self._cache, weights.data_ptr(): (weights, lin)}
        return lin

    def forward(self, activations: torch.Tensor, weights: torch.Tensor, scales: torch.Tensor, zeros: Optional[torch.Tensor] = None,
                group_size: int = 128) -> torch.Tensor:
        x = activations.reshape(-1, activations.shape[-1])
        lin = self._linear(weights, scales, zeros, group_size, x.shape[-1], self.device or x.device)
        y = lin(x.to(torch.bfloat16) if x.device.type == "cuda" else x)
        return y.to(activations.dtype).reshape(*activations.shape[:-1], -1)

    __call__ = forward


# ------------------------------------------------------------------------------------------------ activation functions
def silu_metal(x: torch.Tensor) -> torch.Tensor:
    return torch.nn.functional.silu(x)


def gelu_metal(x: torch.Tensor) -> torch.Tensor:
    return torch.nn.functional.gelu(x)


def relu_metal(x: torch.Tensor) -> torch.Tensor:
    return torch.relu(x)


def swiglu_fused_metal(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up``; bf16 CUDA tensors go through the fused kernel (one read of each input, one write)."""
    if gate.shape != up.shape:
        raise ValueError(f"gate {tuple(gate.shape)} and up {tuple(up.shape)} differ in shape")
    if gate.is_cuda and gate.dtype == torch.bfloat16 and gate.dim() >= 1 and gate.shape[-1] % 8 == 0:
        gu = torch.cat([gate.reshape(-1, gate.shape[-1]), up.reshape(-1, up.shape[-1])], -1)
        return ops.silu_mul(gu).reshape(gate.shape)
    return torch.nn.functional.silu(gate) * up


def geglu_fused_metal(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    if gate.shape != up.shape:
        raise ValueError(f"gate {tuple(gate.shape)} and up {tuple(up.shape)} differ in shape")
    return torch.nn.functional.gelu(gate) * up


def cholesky_decompose(H, regularization: float = 1e-6) -> np.ndarray:
    """Lower Cholesky factor of ``H + regularization * mean(diag) * I`` in float64 (damping grows tenfold until the factorisation
    succeeds).  Reference ``gptq_metal.py:1120``."""
    from .quant.psd import damp_until_cholesky
    Ht = torch.as_tensor(np.asarray(H) if not isinstance(H, torch.Tensor) else H).double()
    Hd, _L32, lam = damp_until_cholesky(Ht, regularization)
    if lam == lam:                       # a plain damping worked: redo the factorisation in float64 on the undamaged input
        Hd = Ht + lam * torch.eye(Ht.shape[-1], dtype=torch.float64, device=Ht.device)
    return torch.linalg.cholesky(Hd.double()).cpu().numpy().astype(np.float64)


# ------------------------------------------------------------------------------------------------ expert weight buffer pool
_EXPERT_POOL: Dict[str, Any] = {"arena": None}


def is_expert_buffer_pool_available() -> bool:
    return _EXPERT_POOL["arena"] is not None


def initialize_expert_buffer_pool(device=None, heap_size: int = 1 << 30) -> bool:
    """One arena (best fit with coalescing, in the native runtime) that expert weight buffers are carved from, so that
    bringing an expert in does not call the device allocator.  ``device``: a torch device or name (the reference passes a
    device pointer; on this platform the slab is an ordinary tensor).  Returns True when a pool exists afterwards.
    Reference ``expert_manager_cpp.py:91``."""
    from .memory import Arena
    if _EXPERT_POOL["arena"] is None:
        dev = torch.device(device) if device is not None and not isinstance(device, int) else torch.device("cuda" if torch.cuda.is_available() else "cpu")
        _EXPERT_POOL["arena"] = Arena(int(heap_size), dev)
    return True


def get_expert_buffer_pool():
    return _EXPERT_POOL["arena"]


def allocate_expert_weight_buffer(size: int) -> torch.Tensor:
    """``size`` bytes from the pool as a ``uint8`` tensor (``arena.free(t)`` returns it)."""
    if _EXPERT_POOL["arena"] is None:
        raise RuntimeError("the expert buffer pool is not initialised (call initialize_expert_buffer_pool first)")
    return _EXPERT_POOL["arena"].alloc((int(size),), torch.uint8, tag="expert")


def clear_expert_buffer_pool() -> None:
    a = _EXPERT_POOL["arena"]
    _EXPERT_POOL["arena"] = None
    if a is not None and hasattr(a, "close"):
        a.close()
