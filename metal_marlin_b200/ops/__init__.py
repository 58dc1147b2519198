"""Op layer: one functional API, two implementations.

CUDA tensors run the hand-written sm_100a kernels in ``_C.so`` (loaded eagerly and
*required* whenever a GPU is present: a missing or stale library raises instead of
falling back).  CPU tensors — and any call made under ``force_reference()`` — run the
PyTorch restatement in ``ops/reference.py``.  Parity: reference
``metal_marlin/kernels_core.py:1830-5370`` (flat python wrappers around Metal
dispatches) and the try/except fallbacks around them.
"""
from __future__ import annotations

import contextlib
import os
from typing import Optional

import torch

from .. import _build
from . import reference as ref
from .weights import FP4ExpertBank, FP4Weight  # noqa: F401

_FORCE_REF = os.environ.get("MMB200_FORCE_TORCH", "0") == "1"
_native_ok = False
GEMV_MAX_M = 32          # dense projections: at or below this many tokens the weight-streaming GEMV path is used
GEMV_FUSED_PROLOGUE_MAX_M = 8   # ... with the residual add + RMSNorm fused into its staging up to this many tokens
ROUTER_GEMM_MIN_T = 64   # above this many tokens the gate logits come from the bf16 tcgen05 GEMM
MOE_GEMV_MAX_T = 8       # MoE: per-(token, slot) streaming up to this many tokens (measured: the expert-sorted kernel wins from 9)
MOE_GROUPED_GEMV_MAX_T = 128   # ... expert-sorted 8-row tiles on the streaming kernel up to here, grouped tcgen05 GEMMs above
GEMV_LIMITS = {}         # (out_features, in_features) -> tuned GEMV_MAX_M of that shape (installed by autotune.apply_config)
MOE_TOKEN_TILES = []     # sorted (tokens, token tile): tuned tile of the grouped GEMM, nearest measured token count wins
GROUPED_GEMV_TUNE = [0, 0, 0, 0]   # (wpt, units per item) of the gate-up and the down launch; 0 = launcher's choice
# Diagnostic switch: route every shape through the weight-streaming kernels (no tcgen05 GEMM).
NO_TCGEN05 = os.environ.get("MMB200_NO_TCGEN05", "0") == "1"


def native_available() -> bool:
    global _native_ok
    if _native_ok:
        return True
    if not torch.cuda.is_available():
        return False
    _build.load(require=True)
    _native_ok = True
    return True


@contextlib.contextmanager
def force_reference(flag: bool = True):
    """Run ops through the PyTorch restatement even on CUDA tensors (tests, baselines)."""
    global _FORCE_REF
    old = _FORCE_REF
    _FORCE_REF = flag
    try:
        yield
    finally:
        _FORCE_REF = old


# Calibration capture: when set, called as ``fn(kind, W, x, ids)`` with the effective input of every quantized
# matrix product (``kind`` "linear" | "moe_gate_up" | "moe_down"; ``x`` after the fused add + norm).
_capture = None


def set_capture(fn) -> None:
    global _capture
    _capture = fn


def _use_native(t: torch.Tensor) -> bool:
    return t.is_cuda and not _FORCE_REF and native_available()


_status = {}


def gemm_status(device) -> torch.Tensor:
    """Per-device int32[4] status word written by kernels whose bounded waits expire."""
    key = str(device)
    if key not in _status:
        _status[key] = torch.zeros(4, dtype=torch.int32, device=device)
        if torch.device(device).type == "cuda" and native_available():
            torch.ops.mmb200.set_status_word(_status[key])     # kernels without a status argument report here too
    return _status[key]


def clear_status(device) -> None:
    gemm_status(device).zero_()


def check_status(device) -> int:
    """Host read of the status word (synchronises).  0 = no wait timed out."""
    return int(gemm_status(device)[0].item())


class _NativeOps:
    """``K.mmb200.<op>(...)`` forwards to ``torch.ops.mmb200.<op>`` and counts kernel launches, so
    benchmarks can report how many of this library's kernels ran inside a timed region."""
    KERNELS_PER_CALL = {"paged_decode": 1, "decode_merge": 1}

    def __init__(self):
        self.launches = 0
        self._cache = {}

    def __getattr__(self, name):
        if name.startswith("_") or name in ("launches", "mmb200"):
            raise AttributeError(name)
        fn = getattr(torch.ops.mmb200, name)
        n = self.KERNELS_PER_CALL.get(name, 1)

        def call(*args):
            self.launches += n
            return fn(*args)

        self.__dict__[name] = call
        return call


class _K:
    mmb200 = _NativeOps()


K = _K()


def launch_count() -> int:
    """Number of native kernel launches issued through this module so far."""
    return K.mmb200.launches


def rmsnorm(x, w, eps=1e-6, *, delta=None, resid_out=None, out=None):
    if not _use_native(x):
        return ref.rmsnorm(x, w, eps, delta, resid_out, out)
    if out is None:
        out = torch.empty_like(x)
    K.mmb200.rmsnorm(x, delta, w, out, resid_out, eps)
    return out


def layernorm(x, w=None, b=None, eps=1e-5, *, delta=None, resid_out=None, out=None):
    """LayerNorm over the last axis (vision encoders, Mamba / RWKV blocks).  ``x`` of any leading shape; bf16 on CUDA runs the
    kernel in ``csrc/elementwise.cu``; parity: reference ``src/layernorm.metal:149``."""
    shape = x.shape
    x2 = x.reshape(-1, shape[-1])
    if not (_use_native(x2) and x2.dtype == torch.bfloat16 and shape[-1] % 2 == 0 and x2.stride(1) == 1):
        v = x2.to(torch.float32)
        if delta is not None:
            v = (v + delta.reshape(-1, shape[-1]).to(torch.float32)).to(x.dtype).to(torch.float32)
            if resid_out is not None:
                resid_out.copy_(v.to(resid_out.dtype).view_as(resid_out))
        y = torch.nn.functional.layer_norm(v, (shape[-1],), None if w is None else w.float(), None if b is None else b.float(), eps).to(x.dtype)
        if out is not None:
            out.copy_(y.view_as(out))
            return out
        return y.view(shape)
    if out is None:
        out = torch.empty_like(x2)
    d2 = None if delta is None else delta.reshape(-1, shape[-1]).contiguous()
    K.mmb200.layernorm(x2 if d2 is None else x2.contiguous(), d2, None if w is None else w.to(torch.bfloat16), None if b is None else b.to(torch.bfloat16),
                       out.view(-1, shape[-1]), resid_out, eps)
    return out.view(shape)


GEMV_BIG_WEIGHT = 24_000_000     # weights of this many elements or more leave the streaming kernel at GEMV_BIG_MAX_M tokens already
GEMV_BIG_MAX_M = 24              # (measured in whole Qwen3-4B steps: the tcgen05 GEMM wins at 32 tokens, 3942 vs 3584 tok/s, and loses at 24)


def _gemv_limit(W) -> int:
    if GEMV_LIMITS:
        lim = GEMV_LIMITS.get((W.out_features, W.in_features))
        if lim is not None:
            return lim
    if W.out_features * W.in_features >= GEMV_BIG_WEIGHT:
        return min(GEMV_MAX_M, GEMV_BIG_MAX_M)
    return GEMV_MAX_M


def linear(x, W: FP4Weight, *, delta=None, norm_w=None, eps=1e-6, resid_out=None, act=0, bias=None, out_add=None,
           out=None, token_tile=0, tpx=None, ag_wait=None, _rotated=False):
    """``out = epilogue( prologue(x) @ dequant(W)^T )``; prologue = optional residual add + RMSNorm,
    epilogue = optional bias, SwiGLU over the two row halves (``act=1``), residual add.

    ``ag_wait``: ``x`` is a gathered buffer whose rows are still arriving from the tensor-parallel peers; the GEMM
    waits per token tile for the owners of the rows (an object with ``.wait`` descriptor and ``.ensure()``)."""
    if ag_wait is not None:
        direct = (delta is None and norm_w is None and _use_native(x) and not getattr(W, "is_generic", False) and _capture is None
                  and x.shape[0] > _gemv_limit(W) and not NO_TCGEN05 and x.is_contiguous() and x.shape[1] == W.in_features)
        if not direct:
            ag_wait.ensure()
            ag_wait = None
    if getattr(W, "is_generic", False):
        from . import generic
        return generic.linear(x, W, delta=delta, norm_w=norm_w, eps=eps, resid_out=resid_out, act=act, bias=bias,
                              out_add=out_add, out=out)
    hb = getattr(W, "hadamard_block", 0)
    if hb and not _rotated:
        # weight stored in a block-Hadamard-rotated basis (MR-GPTQ): y = W_rot . H(norm(x + delta)); the add + norm cannot
        # stay fused in the streaming kernel's prologue because the rotation sits between them and the product
        assert tpx is None or (delta is None and norm_w is None)
        xin = x[:, : W.in_features]
        if delta is not None or norm_w is not None:
            xin = rmsnorm(x, norm_w, eps, delta=delta, resid_out=resid_out) if norm_w is not None else _add(x, delta, resid_out)
            xin = xin[:, : W.in_features]
        xin = hadamard(xin.contiguous(), hb)
        return linear(xin, W, act=act, bias=bias, out_add=out_add, out=out, token_tile=token_tile, tpx=tpx, _rotated=True)
    if _capture is not None:
        _capture("linear", W, ref.add_norm(x[:, : W.in_features], None if delta is None else delta[:, : W.in_features], norm_w, eps), None)
    if not _use_native(x):
        return ref.linear(x, W, delta=delta, norm_w=norm_w, eps=eps, resid_out=resid_out, act=act, bias=bias,
                          out_add=out_add, out=out)
    M = x.shape[0]
    n_out = W.out_features // 2 if act == 1 else W.out_features
    if out is None:
        out = torch.empty(M, n_out, dtype=torch.bfloat16, device=x.device)
    if M <= _gemv_limit(W) or tpx is not None or NO_TCGEN05:      # the in-kernel exchange exists on the streaming kernel only
        if M > GEMV_FUSED_PROLOGUE_MAX_M and tpx is None and delta is not None:
            # every CTA of the streaming kernel stages all its token rows: with many rows the residual add (+ norm, + the
            # residual write) is cheaper done once in its own launch than repeated by every CTA; a norm alone stays fused
            xin = torch.empty(M, x.shape[1], dtype=torch.bfloat16, device=x.device)
            if norm_w is not None:
                K.mmb200.rmsnorm(x, delta, norm_w, xin, resid_out, eps)
            else:
                K.mmb200.add(x.contiguous(), delta.contiguous(), xin)
                if resid_out is not None:
                    resid_out.copy_(xin)
            x, delta, norm_w, resid_out = xin, None, None, None
        if (x.data_ptr() & 15) or (x.stride(0) & 7) or (W.in_features & 7):
            x = x[:, : W.in_features].contiguous()      # the kernel stages activations with 16-byte loads
            if delta is not None:
                delta = delta[:, : W.in_features].contiguous()
        K.mmb200.fp4_gemv(x, W.qtile, W.stile, out, W.out_features, W.in_features, W.group_size, delta, norm_w,
                          resid_out, eps, act, bias, out_add, tpx)
        return out
    assert tpx is None, "the in-kernel tensor-parallel exchange is a decode (small-M) path"
    # tensor-core path: prologue/epilogue pieces run as their own (memory-bound) kernels
    xin = x
    if norm_w is not None or delta is not None:
        xin = torch.empty(M, W.in_features, dtype=torch.bfloat16, device=x.device)
        if norm_w is not None:
            K.mmb200.rmsnorm(x, delta, norm_w, xin, resid_out, eps)
        else:
            K.mmb200.add(x.contiguous(), delta.contiguous(), xin)
            if resid_out is not None:
                resid_out.copy_(xin)
    elif not xin.is_contiguous() or xin.shape[1] != W.in_features:
        xin = xin[:, : W.in_features].contiguous()
    if act == 1 and ag_wait is None and W.out_features % 128 == 0 and bias is None:
        # SwiGLU in the GEMM's epilogue: the gate | up product never goes through memory
        K.mmb200.fp4_gemm_swiglu(xin, W.qtile, W.stile, out, W.out_features, W.group_size, gemm_status(x.device))
        if out_add is not None:
            out += out_add
        return out
    y = out if act == 0 else torch.empty(M, W.out_features, dtype=torch.bfloat16, device=x.device)
    if ag_wait is not None:
        K.mmb200.fp4_gemm_ag(xin, W.qtile, W.stile, y, W.out_features, W.group_size, gemm_status(x.device), ag_wait.wait)
    else:
        K.mmb200.fp4_gemm(xin, W.qtile, W.stile, y, W.out_features, W.group_size, gemm_status(x.device))
    if bias is not None:
        y += bias
    if act == 1:
        K.mmb200.silu_mul(y, out)
    if out_add is not None:
        out += out_add
    return out


def _add(x, delta, resid_out=None):
    y = (x.to(torch.float32) + delta.to(torch.float32)).to(x.dtype)
    if resid_out is not None:
        resid_out.copy_(y)
    return y


def bf16_linear(x, w, *, delta=None, norm_w=None, eps=1e-6, out_dtype=torch.bfloat16, out=None, tpx=None):
    if not _use_native(x):
        return ref.bf16_linear(x, w, delta=delta, norm_w=norm_w, eps=eps, out_dtype=out_dtype, out=out)
    M = x.shape[0]
    if out is None:
        out = torch.empty(M, w.shape[0], dtype=out_dtype, device=x.device)
    if M <= 8 or tpx is not None or w.shape[1] % 64 != 0:
        K.mmb200.bf16_gemv(x, w, out, delta, norm_w, eps, tpx)      # weight-streaming: every weight row read once per 4 tokens
        return out
    # more tokens: the tcgen05 GEMM streams the weight once for all of them (A operand by TMA, fp32 in TMEM)
    xin = x
    if norm_w is not None or delta is not None:
        xin = torch.empty_like(x)
        if norm_w is not None:
            K.mmb200.rmsnorm(x, delta, norm_w, xin, None, eps)
        else:
            K.mmb200.add(x.contiguous(), delta.contiguous(), xin)
    elif not xin.is_contiguous():
        xin = xin.contiguous()
    K.mmb200.bf16_gemm(xin, w, out, gemm_status(x.device))
    return out


def silu_mul(gu, out=None):
    if not _use_native(gu):
        return ref.silu_mul(gu, out)
    if out is None:
        out = torch.empty(gu.shape[0], gu.shape[1] // 2, dtype=gu.dtype, device=gu.device)
    K.mmb200.silu_mul(gu, out)
    return out


def embedding(table, ids, out=None):
    if not _use_native(table):
        return ref.embedding(table, ids, out)
    ids = ids.reshape(-1).contiguous()
    if out is None:
        out = torch.empty(ids.numel(), table.shape[1], dtype=table.dtype, device=table.device)
    K.mmb200.embedding(table, ids, out)
    return out


def rope(q, k, positions, inv_freq, Hq, Hk, D, rot_dim, interleaved=False, mscale=1.0):
    if not _use_native(q):
        return ref.rope(q, k, positions, inv_freq, Hq, Hk, D, rot_dim, interleaved, mscale)
    K.mmb200.rope(q, k, positions, inv_freq, Hq, Hk, D, rot_dim, interleaved, mscale)
    return q, k


KV_FORMATS = {"fp8": 0, "int8": 1, "fp4": 2, "int4": 3}
_KV_RANGE = {0: 448.0, 1: 127.0, 2: 6.0, 3: 7.0}
_E2M1_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
_E2M1_MIDPOINTS = (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0)


class FP8KV:
    """Quantized paged KV pool with one fp32 scale per cached row: ``data`` uint8 ``[num_slots, Hkv, W]`` (GQA) or
    ``[num_slots, W]`` (MLA latent) and ``scale`` fp32 ``[num_slots, Hkv | 1]``.  ``fmt``: ``"fp8"`` (E4M3, scale = row amax / 448;
    the default the class is named for), ``"int8"`` (amax / 127), ``"fp4"`` (E2M1, amax / 6) or ``"int4"`` (amax / 7); the
    8-bit formats hold one byte per value (``W = D``), the 4-bit formats two values per byte, even element in the low nibble
    (``W = D / 2``).  Indexing with slot ids returns the de-quantized bf16 rows, so code that gathers rows from a bf16 pool
    works unchanged.

    Parity: reference ``metal_marlin/kv_cache.py`` (fp8 / int8 / fp4 cache modes) and ``paged_attention_v1_fp8``,
    ``paged_attention_v1_fp4`` ``:670``, ``paged_attention_v1_int4`` ``:885`` (``src/paged_attention.metal``: packed codes with
    per-token-per-head scales)."""

    def __init__(self, num_slots: int, row_shape, device, fmt: str = "fp8"):
        row_shape = tuple(row_shape)
        self.fmt = fmt
        self.fmt_code = KV_FORMATS[fmt]
        self.four_bit = self.fmt_code >= 2
        self.width = row_shape[-1]                                   # values per row
        if self.four_bit and self.width % 32:
            raise ValueError("4-bit KV rows must hold a multiple of 32 values")
        stored = row_shape[:-1] + (self.width // 2 if self.four_bit else self.width,)
        self.data = torch.zeros(num_slots, *stored, dtype=torch.uint8, device=device)
        self.scale = torch.ones(num_slots, row_shape[0] if len(row_shape) == 2 else 1, dtype=torch.float32, device=device)

    device = property(lambda self: self.data.device)
    dtype = torch.uint8

    @property
    def shape(self):
        return self.data.shape[:-1] + (self.width,)

    def view(self, *shape):
        return self

    def numel(self):
        return self.data.numel() * (2 if self.four_bit else 1)

    def element_size(self):
        return 1

    def nbytes(self) -> int:
        return self.data.numel() + self.scale.numel() * 4

    # ---- PyTorch restatement of the kernels' quantizer and de-quantizer (kv_quant.cuh)
    def _encode(self, x: torch.Tensor) -> torch.Tensor:
        """``x`` = value / row scale -> integer codes (uint8, one per value)."""
        c = self.fmt_code
        if c == 0:
            return x.clamp(-448.0, 448.0).to(torch.float8_e4m3fn).view(torch.uint8)
        if c == 1:
            return torch.round(x.clamp(-127.0, 127.0)).to(torch.int16).bitwise_and(0xFF).to(torch.uint8)
        if c == 3:
            return torch.round(x.clamp(-7.0, 7.0)).to(torch.int16).bitwise_and(0xF).to(torch.uint8)
        mag = torch.bucketize(x.abs(), torch.tensor(_E2M1_MIDPOINTS, device=x.device, dtype=x.dtype), right=True)
        return (mag + 8 * (x < 0).to(mag.dtype)).to(torch.uint8)

    def _decode(self, codes: torch.Tensor) -> torch.Tensor:
        c = self.fmt_code
        if c == 0:
            return codes.view(torch.float8_e4m3fn).float()
        if c == 1:
            return codes.view(torch.int8).float()
        n = codes.to(torch.int16)
        if c == 3:
            return torch.where(n >= 8, n - 16, n).float()
        tab = torch.tensor(_E2M1_VALUES, device=codes.device, dtype=torch.float32)
        v = tab[(n & 7).long()]
        return torch.where(n >= 8, -v, v)

    def store(self, slots, rows):
        """Quantize ``rows`` (float ``[n, ...row_shape]``, bf16-rounded first) into the given slots."""
        r = rows.to(torch.bfloat16).float()
        amax = r.abs().amax(-1)
        sc = torch.where(amax > 0, amax / _KV_RANGE[self.fmt_code], torch.ones_like(amax))
        q = self._encode(r * (1.0 / sc).unsqueeze(-1))
        if self.four_bit:
            q = q[..., 0::2] | (q[..., 1::2] << 4)
        self.data[slots] = q
        self.scale[slots] = sc.reshape(sc.shape[0], -1)

    def __getitem__(self, idx):
        d = self.data[idx]
        if self.four_bit:
            d = torch.stack([d & 0xF, d >> 4], -1).flatten(-2)
        d = self._decode(d)
        sc = self.scale[idx]
        return (d * (sc.unsqueeze(-1) if d.dim() == sc.dim() + 1 else sc)).to(torch.bfloat16)

    def dequantize(self):
        return self[torch.arange(self.data.shape[0], device=self.data.device)]


QuantKV = FP8KV


def kv_copy_rows(pool, dst, src) -> None:
    """``pool[dst] = pool[src]`` (slices or index tensors) for bf16 pools and FP8 pools alike (copy-on-write of cache
    blocks, compaction of accepted speculative rows)."""
    if isinstance(pool, FP8KV):
        pool.data[dst] = pool.data[src].clone()
        pool.scale[dst] = pool.scale[src].clone()
    else:
        pool[dst] = pool[src].clone()


def _ref_cache_write(fn, pool_pairs, slots, n_tok):
    """Runs a reference cache-writing op against scratch bf16 pools with identity slots, then quantizes the written rows
    into the FP8 pools."""
    ident = torch.where(slots >= 0, torch.arange(n_tok, device=slots.device), torch.full_like(slots, -1))
    tmps = [torch.zeros(n_tok, *p.shape[1:], dtype=torch.bfloat16, device=p.data.device) for p in pool_pairs]
    r = fn(ident, tmps)
    ok = slots >= 0
    for p, t in zip(pool_pairs, tmps):
        p.store(slots[ok], t[ok])
    return r


def qk_norm_rope_cache(q, k, v, qn_w, kn_w, positions, inv_freq, slots, k_pool, v_pool, Hq, Hk, D, eps, interleaved=False):
    if isinstance(k_pool, FP8KV):
        if not _use_native(q):
            _ref_cache_write(lambda sl, t: ref.qk_norm_rope_cache(q, k, v, qn_w, kn_w, positions, inv_freq, sl, t[0], t[1], Hq, Hk, D, eps,
                                                                  interleaved), [k_pool, v_pool], slots, q.shape[0])
            return q
        K.mmb200.qk_norm_rope_cache_fp8(q, k, v, qn_w, kn_w, positions, inv_freq, slots, k_pool.data, v_pool.data, k_pool.scale,
                                        v_pool.scale, Hq, Hk, D, eps, interleaved, k_pool.fmt_code)
        return q
    if not _use_native(q):
        return ref.qk_norm_rope_cache(q, k, v, qn_w, kn_w, positions, inv_freq, slots, k_pool, v_pool, Hq, Hk, D, eps,
                                      interleaved)
    K.mmb200.qk_norm_rope_cache(q, k, v, qn_w, kn_w, positions, inv_freq, slots, k_pool, v_pool, Hq, Hk, D, eps, interleaved)
    return q


def mla_prep(q, kva, w_ukT, kv_norm_w, positions, inv_freq, slots, q_full, cache, H, dn, dr, R, eps, mscale=1.0,
             interleaved=True, skip_absorb=False):
    """``skip_absorb``: only RoPE the query's rope slice into ``q_full[..., R:]`` and write the new latent rows (prefill
    attends in the non-absorbed form and never needs ``q_full[..., :R]``)."""
    if isinstance(cache, FP8KV):
        if not _use_native(q):
            _ref_cache_write(lambda sl, t: ref.mla_prep(q, kva, w_ukT, kv_norm_w, positions, inv_freq, sl, q_full, t[0], H, dn, dr, R, eps,
                                                        mscale, interleaved), [cache], slots, q.shape[0])
            return q_full
        K.mmb200.mla_prep_fp8(q, kva, w_ukT, kv_norm_w, positions, inv_freq, slots, q_full, cache.data, cache.scale.view(-1), H, dn, dr, R,
                              eps, mscale, interleaved, skip_absorb, cache.fmt_code)
        return q_full
    if not _use_native(q):
        return ref.mla_prep(q, kva, w_ukT, kv_norm_w, positions, inv_freq, slots, q_full, cache, H, dn, dr, R, eps,
                            mscale, interleaved)
    K.mmb200.mla_prep(q, kva, w_ukT, kv_norm_w, positions, inv_freq, slots, q_full, cache, H, dn, dr, R, eps, mscale,
                      interleaved, skip_absorb)
    return q_full


def kv_fp8_rows(pool: "FP8KV", block_tables, ctx_lens, cu_k, total: int, max_ctx: int, block_size: int):
    """Contiguous bf16 ``[total, Hkv, D]`` rows of the sequences described by ``block_tables`` / ``ctx_lens``."""
    Hkv, D = (pool.data.shape[1] if pool.data.dim() == 3 else 1), pool.width
    out = torch.empty(total, Hkv, D, dtype=torch.bfloat16, device=pool.data.device)
    if _use_native(pool.data) and D % 8 == 0:
        K.mmb200.kv_fp8_gather(pool.data, pool.scale, block_tables, ctx_lens, cu_k, out, Hkv, D, block_size, max_ctx, pool.fmt_code)
        return out
    cl, ck = ctx_lens.tolist(), cu_k.tolist()
    for b, n in enumerate(cl):
        tok = torch.arange(n, device=pool.data.device)
        slots = block_tables[b, tok // block_size].long() * block_size + tok % block_size
        out[ck[b]: ck[b] + n] = pool[slots].view(n, Hkv, D)
    return out


def default_splits(batch: int, n_kv_heads: int, max_ctx: int, sm_count: int = 148, mla_latent: bool = False) -> int:
    """Split-KV factor so that batch * kv_heads * splits covers the SMs (at least one 64-token tile per split).
    ``mla_latent``: the 576 / 512 latent shape has a two-CTAs-per-SM kernel variant (32-token tiles) that the launcher
    picks when the grid exceeds the SM count, so once a batch leaves four splits per sequence or fewer the target is two
    CTAs per SM."""
    tiles = max(1, (max_ctx + 63) // 64)
    bh = max(1, batch * n_kv_heads)
    want = max(1, sm_count // bh)
    if mla_latent and want <= 4 and bh <= 2 * sm_count:
        want = max(1, (2 * sm_count) // bh)
    return int(max(1, min(want, tiles, 64)))


def paged_attention(q, k_pool, v_pool, block_tables, ctx_lens, *, Hq, Hkv, dqk, dv, block_size, scale, window=0,
                    splits=None, w_uv=None, workspace=None, out=None, max_ctx=None):
    """Decode attention over a paged pool.  With ``w_uv [Hq, dvo, dv]`` the merged latent output is
    up-projected per head (MLA).  Returns bf16 ``[B, Hq, dvo or dv]``."""
    B = ctx_lens.numel()
    dvo = w_uv.shape[1] if w_uv is not None else dv
    fp8 = isinstance(k_pool, FP8KV)
    if not _use_native(q):
        if fp8:      # the oracle attends over the de-quantized pools
            k_pool, v_pool = k_pool.dequantize(), (v_pool.dequantize() if v_pool is not None else None)
        o = ref.paged_attention(q, k_pool, v_pool, block_tables, ctx_lens, Hq, Hkv, dqk, dv, block_size, scale, window)
        if w_uv is not None:
            o = ref.mla_up(o, w_uv)
        if out is not None:
            out.copy_(o.view_as(out))
            return out
        return o
    if splits is None:
        if max_ctx is None:
            max_ctx = block_tables.shape[1] * block_size
        splits = default_splits(B, Hkv, max_ctx, mla_latent=(v_pool is None and dqk == 576 and dv == 512 and not fp8))
    if workspace is None:
        part_o = torch.empty(B * Hq * splits * dv, dtype=torch.float32, device=q.device)
        part_ml = torch.empty(B * Hq * splits * 2, dtype=torch.float32, device=q.device)
    else:
        part_o, part_ml = workspace
    if out is None:
        out = torch.empty(B, Hq, dvo, dtype=torch.bfloat16, device=q.device)
    gemm_status(q.device)        # registers the device's status word on first use: the kernel's bounded waits report there
    if fp8:
        K.mmb200.paged_decode_fp8(q, k_pool.data, None if v_pool is None else v_pool.data, k_pool.scale,
                                  None if v_pool is None else v_pool.scale, block_tables, ctx_lens, part_o, part_ml, Hq, Hkv, dqk, dv,
                                  block_size, splits, scale, window, k_pool.fmt_code)
    else:
        K.mmb200.paged_decode(q, k_pool, v_pool, block_tables, ctx_lens, part_o, part_ml, Hq, Hkv, dqk, dv, block_size,
                              splits, scale, window)
    K.mmb200.decode_merge(part_o, part_ml, w_uv, out, B, Hq, dv, dvo, splits)
    return out


def moe_router(x, w, *, delta=None, norm_w=None, eps=1e-6, resid_out=None, bias=None, topk=4, scoring=0, renorm=True,
               routed_scale=1.0, n_group=1, topk_group=1, ids=None, weights=None, logits_out=None, counts=None,
               tpx=None, ag_wait=None):
    if ag_wait is not None:
        direct = (_use_native(x) and x.shape[0] > ROUTER_GEMM_MIN_T and tpx is None and w.shape[1] % 64 == 0 and x.is_contiguous()
                  and norm_w is None and delta is None)
        if not direct:
            ag_wait.ensure()
            ag_wait = None
    if not _use_native(x):
        i, wt, lg = ref.moe_router(x, w, delta=delta, norm_w=norm_w, eps=eps, resid_out=resid_out, bias=bias, topk=topk,
                                   scoring=scoring, renorm=renorm, routed_scale=routed_scale, n_group=n_group,
                                   topk_group=topk_group)
        if ids is not None:
            ids.copy_(i)
            weights.copy_(wt)
            i, wt = ids, weights
        if logits_out is not None:
            logits_out.copy_(lg)
        if counts is not None:
            counts += torch.bincount(i.reshape(-1).long(), minlength=counts.numel()).to(counts.dtype)
        return i, wt
    T = x.shape[0]
    if ids is None:
        ids = torch.empty(T, topk, dtype=torch.int32, device=x.device)
        weights = torch.empty(T, topk, dtype=torch.float32, device=x.device)
    if T > ROUTER_GEMM_MIN_T and tpx is None and w.shape[1] % 64 == 0 and x.is_contiguous():
        # prefill: add + norm kernel, gate logits on the tensor cores, then one warp per token scores and selects
        xin = torch.empty_like(x)
        if norm_w is not None:
            K.mmb200.rmsnorm(x, delta, norm_w, xin, resid_out, eps)
        elif delta is not None:
            K.mmb200.add(x, delta.contiguous(), xin)
            if resid_out is not None:
                resid_out.copy_(xin)
        else:
            xin = x
        lg = logits_out if logits_out is not None else torch.empty(T, w.shape[0], dtype=torch.float32, device=x.device)
        if ag_wait is not None:      # gathered rows still arriving: the GEMM waits per token tile
            K.mmb200.bf16_gemm_ag(xin, w, lg, gemm_status(x.device), ag_wait.wait)
        else:
            K.mmb200.bf16_gemm(xin, w, lg, gemm_status(x.device))
        K.mmb200.moe_select(lg, bias, ids, weights, counts, topk, scoring, renorm, routed_scale, n_group, topk_group)
        return ids, weights
    K.mmb200.moe_router(x, w, delta, norm_w, resid_out, bias, ids, weights, logits_out, counts, topk, eps, scoring,
                        renorm, routed_scale, n_group, topk_group, tpx)
    return ids, weights


def moe_select(logits, *, bias=None, topk=4, scoring=0, renorm=True, routed_scale=1.0, n_group=1, topk_group=1, counts=None):
    """Expert choice from gate logits fp32 ``[T, E]`` (softmax or sigmoid scoring, optional group-limited top-k, optional
    renormalisation): ``(ids int32 [T, topk], weights fp32 [T, topk])``; ``counts`` int32 ``[E]`` accumulates the load.  One
    warp per token on the GPU.  The logits may come from any gate: bf16 GEMM, INT8 router (``moe/router_int8.py``)."""
    if not _use_native(logits):
        ids, wts = ref.moe_select(logits, bias=bias, topk=topk, scoring=scoring, renorm=renorm, routed_scale=routed_scale,
                                  n_group=n_group, topk_group=topk_group)
        if counts is not None:
            counts += torch.bincount(ids.reshape(-1).long(), minlength=counts.numel()).to(counts.dtype)
        return ids, wts
    T = logits.shape[0]
    ids = torch.empty(T, topk, dtype=torch.int32, device=logits.device)
    weights = torch.empty(T, topk, dtype=torch.float32, device=logits.device)
    K.mmb200.moe_select(logits.to(torch.float32).contiguous(), bias, ids, weights, counts, topk, scoring, renorm, routed_scale,
                        n_group, topk_group)
    return ids, weights


def moe_gate_up(x, bank: FP4ExpertBank, ids, *, n_shared=0, shared_base=0, norm_w=None, eps=1e-6, out=None):
    if not _use_native(x):
        return ref.moe_gate_up(x, bank, ids, n_shared=n_shared, shared_base=shared_base, norm_w=norm_w, eps=eps, out=out)
    T, topk = ids.shape
    S = topk + n_shared
    if out is None:
        out = torch.empty(T * S, bank.out_features // 2, dtype=torch.bfloat16, device=x.device)
    K.mmb200.fp4_moe_gemv(x, bank.qtile, bank.stile, out, bank.out_features, bank.in_features, bank.group_size, 1, ids,
                          None, n_shared, shared_base, norm_w, eps, 1, None, None)
    return out


def moe_down(h, bank: FP4ExpertBank, ids, weights, *, n_shared=0, shared_base=0, out_add=None, out=None, tpx=None):
    if not _use_native(h):
        return ref.moe_down(h, bank, ids, weights, n_shared=n_shared, shared_base=shared_base, out_add=out_add, out=out)
    T = ids.shape[0]
    if out is None:
        out = torch.empty(T, bank.out_features, dtype=torch.bfloat16, device=h.device)
    K.mmb200.fp4_moe_gemv(h, bank.qtile, bank.stile, out, bank.out_features, bank.in_features, bank.group_size, 2, ids,
                          weights, n_shared, shared_base, None, 0.0, 0, out_add, tpx)
    return out


def tp_argmax(logits, vocab_offset: int, tpx, out=None):
    """Vocab-parallel greedy head: every rank ends with the global arg-max (native path only)."""
    if out is None:
        out = torch.empty(logits.shape[0], dtype=torch.int64, device=logits.device)
    K.mmb200.tp_argmax(logits, out, int(vocab_offset), tpx)
    return out


def argmax(logits, out=None):
    if not _use_native(logits):
        r = logits.argmax(-1)
        if out is not None:
            out.copy_(r)
            return out
        return r
    if out is None:
        out = torch.empty(logits.shape[0], dtype=torch.int64, device=logits.device)
    K.mmb200.argmax(logits, out)
    return out


def sample(logits, *, temperature=None, top_k=None, top_p=None, min_p=None, history=None, rep_penalty=None, seed=0,
           offset=0, out=None, out_logprob=None, generator=None, offset_dev=None, seed_dev=None):
    """Per-row parameters are tensors on the logits' device (None = feature off).  ``seed_dev`` (int64 ``[B]``) gives
    every row its own Philox key and, being device memory, can change between replays of a captured graph."""
    if not _use_native(logits):
        ids, lp = ref.sample(logits, temperature=temperature, top_k=top_k, top_p=top_p, min_p=min_p, history=history,
                             rep_penalty=rep_penalty, generator=generator)
        if out is not None:
            out.copy_(ids)
            ids = out
        if out_logprob is not None:
            out_logprob.copy_(lp)
        return ids
    if out is None:
        out = torch.empty(logits.shape[0], dtype=torch.int64, device=logits.device)
    K.mmb200.sample(logits, out, out_logprob, temperature, top_k, top_p, min_p, history, rep_penalty, int(seed), int(offset),
                    offset_dev, seed_dev)
    return out


def bf16_gemm(x, w, out=None, out_dtype=torch.bfloat16):
    """tcgen05 GEMM ``out[.., M, N] = x[.., M, K] @ w[.., N, K]^T`` (bf16 operands by TMA, fp32 in TMEM)."""
    if not _use_native(x):
        y = torch.matmul(x.to(torch.float32), w.to(torch.float32).transpose(-1, -2)).to(out_dtype)
        if out is not None:
            out.copy_(y)
            return out
        return y
    batched = x.dim() == 3 or w.dim() == 3
    nb = x.shape[0] if x.dim() == 3 else (w.shape[0] if w.dim() == 3 else 1)
    shape = (nb, x.shape[-2], w.shape[-2]) if batched else (x.shape[-2], w.shape[-2])
    if out is None:
        out = torch.empty(shape, dtype=out_dtype, device=x.device)
    K.mmb200.bf16_gemm(x, w, out, gemm_status(x.device))
    return out


def _build_tile_list(flat_ids: torch.Tensor, num_experts: int, token_tile: int):
    """Device-side (no host sync) construction of the grouped-GEMM work list.
    Returns (order, tile_expert, tile_row0, tile_rows, n_tiles)."""
    n = flat_ids.numel()
    order = torch.argsort(flat_ids, stable=True)
    # scatter_add instead of bincount: no host sync, so the whole routine is CUDA-graph capturable
    counts = torch.zeros(num_experts, dtype=torch.int64, device=flat_ids.device).scatter_add_(
        0, flat_ids, torch.ones_like(flat_ids))
    offs = torch.cumsum(counts, 0) - counts
    tiles_per = (counts + token_tile - 1) // token_tile
    tile_end = torch.cumsum(tiles_per, 0)
    tile_start = tile_end - tiles_per
    max_tiles = (n + token_tile - 1) // token_tile + num_experts
    j = torch.arange(max_tiles, device=flat_ids.device)
    e = torch.searchsorted(tile_end, j, right=True).clamp_(max=num_experts - 1)
    local = j - tile_start[e]
    row0 = offs[e] + local * token_tile
    rows = (counts[e] - local * token_tile).clamp_(0, token_tile)
    n_tiles = tile_end[-1:].to(torch.int32)
    return order, e.to(torch.int32), row0.to(torch.int32), rows.to(torch.int32), n_tiles


def _shared_experts(xin, gate_up, down, n_shared, shared_base):
    shared = None
    for j in range(n_shared):
        e = shared_base + j
        hs = linear(xin, gate_up.expert(e), act=1)
        sj = linear(hs, down.expert(e))
        shared = sj if shared is None else shared + sj
    return shared


def _grouped_gemv_ok(bank, act: int) -> bool:
    """Whether the streaming kernel can split this bank's row tiles evenly over the warp groups of a CTA."""
    k = bank.qtile.shape[2] * 64
    k_units = k // max(bank.group_size, 64)
    tps = bank.out_features // (32 if act else 16)
    if bank.out_features % (32 if act else 16):
        return False
    return any(k_units >= w and tps % (8 // w) == 0 for w in (1, 2, 4, 8))


def _moe_forward_grouped_gemv(xin, gate_up, down, ids, weights, n_shared, shared_base, out_add):
    """Medium batches: still bound by weight bytes, but most experts are hit, so tokens are sorted by expert and
    every expert's weights stream once for up to 8 of its rows per tile (gather and routing weight fused into the
    two launches)."""
    T, topk = ids.shape
    n = T * topk
    dev = xin.device
    max_tiles = (n + 7) // 8 + gate_up.num_experts
    order = torch.empty(n, dtype=torch.int32, device=dev)
    inv = torch.empty(n, dtype=torch.int32, device=dev)
    t_e = torch.empty(max_tiles, dtype=torch.int32, device=dev)
    t_r0, t_rows = torch.empty_like(t_e), torch.empty_like(t_e)
    n_tiles = torch.empty(1, dtype=torch.int32, device=dev)
    K.mmb200.moe_group(ids.reshape(-1).contiguous(), gate_up.num_experts, 8, order, inv, t_e, t_r0, t_rows, n_tiles)
    h = torch.empty(n, gate_up.out_features // 2, dtype=torch.bfloat16, device=dev)
    K.mmb200.fp4_grouped_gemv(xin, gate_up.qtile, gate_up.stile, h, gate_up.out_features, gate_up.group_size, 1,
                              t_e, t_r0, t_rows, n_tiles, order, topk, None, GROUPED_GEMV_TUNE[0], GROUPED_GEMV_TUNE[1])
    y = torch.empty(n, down.out_features, dtype=torch.bfloat16, device=dev)
    K.mmb200.fp4_grouped_gemv(h, down.qtile, down.stile, y, down.out_features, down.group_size, 0,
                              t_e, t_r0, t_rows, n_tiles, order, 0, weights.reshape(-1).contiguous(),
                              GROUPED_GEMV_TUNE[2], GROUPED_GEMV_TUNE[3])
    shared = _shared_experts(xin, gate_up, down, n_shared, shared_base)
    out = torch.empty(T, down.out_features, dtype=torch.bfloat16, device=dev)
    K.mmb200.moe_combine(y, inv, shared, None if out_add is None else out_add.contiguous(), out, topk)
    return out


def moe_forward(x, gate_up: FP4ExpertBank, down: FP4ExpertBank, ids, weights, *, n_shared=0, shared_base=0,
                norm_w=None, eps=1e-6, out_add=None, token_tile=0, tpx=None):
    """Whole expert MLP: ``sum_s w_s * down_e(silu(gate_e(x)) * up_e(x))`` over routed + shared experts.

    Few tokens: per-(token, slot) weight-streaming kernels (experts read from device memory ids).
    Many tokens: counting-sort tokens by expert, grouped tcgen05 GEMMs over a device-built tile list."""
    T, topk = ids.shape
    if getattr(gate_up, "is_generic", False):
        from . import generic
        return generic.moe_forward(x, gate_up, ids, weights, n_shared=n_shared, shared_base=shared_base, norm_w=norm_w, eps=eps,
                                   out_add=out_add)
    if getattr(gate_up, "hadamard_block", 0) or getattr(down, "hadamard_block", 0):
        # banks stored in a rotated basis: rotate the (normalised) input once, and the SwiGLU output of every slot
        xin = rmsnorm(x, norm_w, eps) if norm_w is not None else x
        if getattr(gate_up, "hadamard_block", 0):
            xin = hadamard(xin[:, : gate_up.in_features].contiguous(), gate_up.hadamard_block)
        h = moe_gate_up(xin, gate_up, ids, n_shared=n_shared, shared_base=shared_base)
        if getattr(down, "hadamard_block", 0):
            h = hadamard(h.reshape(-1, h.shape[-1])[:, : down.in_features].contiguous(), down.hadamard_block).view(T, -1, down.in_features)
        return moe_down(h, down, ids, weights, n_shared=n_shared, shared_base=shared_base, out_add=out_add, tpx=tpx)
    if _capture is not None:
        # calibration: expose the inputs of both expert projections with the expert of every (token, slot)
        e_all = ids.long()
        if n_shared:
            e_all = torch.cat([e_all, torch.arange(shared_base, shared_base + n_shared, device=ids.device).expand(T, n_shared)], 1)
        _capture("moe_gate_up", gate_up, ref.add_norm(x[:, : gate_up.in_features], None, norm_w, eps), e_all)
        h = moe_gate_up(x, gate_up, ids, n_shared=n_shared, shared_base=shared_base, norm_w=norm_w, eps=eps)
        _capture("moe_down", down, h.view(T, e_all.shape[1], -1)[..., : down.in_features].to(torch.float32), e_all)
        return moe_down(h, down, ids, weights, n_shared=n_shared, shared_base=shared_base, out_add=out_add, tpx=tpx)
    if (not _use_native(x)) or T <= MOE_GEMV_MAX_T or NO_TCGEN05:
        h = moe_gate_up(x, gate_up, ids, n_shared=n_shared, shared_base=shared_base, norm_w=norm_w, eps=eps)
        return moe_down(h, down, ids, weights, n_shared=n_shared, shared_base=shared_base, out_add=out_add, tpx=tpx)
    assert tpx is None
    xin = x
    if norm_w is not None:
        xin = torch.empty_like(x)
        K.mmb200.rmsnorm(x, None, norm_w, xin, None, eps)
    if (T <= MOE_GROUPED_GEMV_MAX_T and xin.shape[1] >= gate_up.qtile.shape[2] * 64
            and gate_up.out_features // 2 == down.qtile.shape[2] * 64 and _grouped_gemv_ok(gate_up, 1)
            and _grouped_gemv_ok(down, 0)):
        return _moe_forward_grouped_gemv(xin, gate_up, down, ids, weights, n_shared, shared_base, out_add)
    st = gemm_status(x.device)
    E_routed = gate_up.num_experts - n_shared
    if not token_tile and MOE_TOKEN_TILES:      # tuned on this GPU: the tile measured best at the nearest token count
        token_tile = min(MOE_TOKEN_TILES, key=lambda e: abs(e[0] - T))[1]
    if not token_tile:      # smallest MMA N tile that holds the average expert load
        avg = T * topk / max(1, E_routed)
        token_tile = 32 if avg <= 24 else (64 if avg <= 48 else (128 if avg <= 160 else 256))
    inter = gate_up.out_features // 2
    n = T * topk
    dev = x.device
    # device-side dispatch: counting sort by expert + tile list (one launch), gather in expert order (one launch)
    max_tiles = (n + token_tile - 1) // token_tile + gate_up.num_experts
    order = torch.empty(n, dtype=torch.int32, device=dev)
    inv = torch.empty(n, dtype=torch.int32, device=dev)
    t_e = torch.empty(max_tiles, dtype=torch.int32, device=dev)
    t_r0, t_rows = torch.empty_like(t_e), torch.empty_like(t_e)
    n_tiles = torch.empty(1, dtype=torch.int32, device=dev)
    K.mmb200.moe_group(ids.reshape(-1).contiguous(), gate_up.num_experts, token_tile, order, inv, t_e, t_r0, t_rows, n_tiles)
    xs = torch.empty(n, gate_up.in_features, dtype=torch.bfloat16, device=dev)
    K.mmb200.moe_gather(xin, order, xs, topk)
    h = torch.empty(n, inter, dtype=torch.bfloat16, device=dev)
    if gate_up.out_features % 128 == 0:
        K.mmb200.fp4_gemm_grouped_swiglu(xs, gate_up.qtile, gate_up.stile, h, gate_up.out_features, gate_up.group_size,
                                         t_e, t_r0, t_rows, n_tiles, token_tile, st)
    else:
        gu = torch.empty(n, gate_up.out_features, dtype=torch.bfloat16, device=dev)
        K.mmb200.fp4_gemm_grouped(xs, gate_up.qtile, gate_up.stile, gu, gate_up.out_features, gate_up.group_size,
                                  t_e, t_r0, t_rows, n_tiles, token_tile, None, st)
        K.mmb200.silu_mul(gu, h)
    y = torch.empty(n, down.out_features, dtype=torch.bfloat16, device=dev)
    # routing weight of every sorted row (dropped pairs, id < 0, are never read by a tile)
    rs = weights.reshape(-1).to(torch.float32).index_select(0, order.clamp_min(0).long()).contiguous()
    K.mmb200.fp4_gemm_grouped(h, down.qtile, down.stile, y, down.out_features, down.group_size,
                              t_e, t_r0, t_rows, n_tiles, token_tile, rs, st)
    shared = _shared_experts(xin, gate_up, down, n_shared, shared_base)
    out = torch.empty(T, down.out_features, dtype=torch.bfloat16, device=dev)
    # combine: un-sort, sum over the token's slots, add the shared expert and the residual input (one launch)
    K.mmb200.moe_combine(y, inv, shared, None if out_add is None else out_add.contiguous(), out, topk)
    return out


# ----------------------------------------------------------------------------------------------------------------
# secondary kernels: Hadamard rotation, trellis weights, codebook (INT4 / INT8 / FP8 / NF4 ...) GEMV, vision
# preprocessing, speculative verification
# ----------------------------------------------------------------------------------------------------------------
def gptq_block(W, Q, Hinv, col_scale, grid, err_rows, i1: int, i2: int):
    """The column-serial part of GPTQ over the lazy block ``[i1, i2)`` (at most 128 columns) as one launch, a warp per
    weight row: writes the quantized columns into ``Q``, adds each row's squared error to ``err_rows`` and returns the
    scaled errors ``E [out, i2 - i1]`` for the update of the columns behind the block.  All tensors fp32 on one CUDA device;
    ``W`` (updated in place), ``Q`` and ``col_scale`` share a row stride.  Bit-identical to the PyTorch loop in
    ``quant.gptq.gptq_quantize`` (plain fp32 roundings).  Parity: reference ``src/cholesky.metal`` (``gptq_update_weights``)."""
    E = torch.empty(W.shape[0], i2 - i1, dtype=torch.float32, device=W.device)
    K.mmb200.gptq_block(W, Q, E, Hinv, col_scale, grid, err_rows, i1, i2 - i1)
    return E


def gptq_block_ok(W, block: int, n_grid: int) -> bool:
    return _use_native(W) and W.dtype == torch.float32 and 1 <= block <= 128 and 2 <= n_grid <= 256


def fp4_quantize_pack(w, group_size: int = 128):
    """Round-to-nearest E2M1 quantization and packing of ``w [out, in]`` (fp32 or bf16) in one pass: returns ``(packed int32
    [out, in / 8], scales fp16 [out, in / group_size])``, the row-packed checkpoint layout.  Equal bit for bit to
    ``formats.fp4.quantize_codes`` followed by ``pack_mmfp4``, which is what runs on the CPU.  Parity: reference
    ``metal_marlin/fp4_metal.py``."""
    lanes = group_size // 8
    if not (_use_native(w) and w.dtype in (torch.float32, torch.bfloat16) and 8 <= group_size <= 128 and lanes & (lanes - 1) == 0
            and group_size % 8 == 0):
        from ..formats import fp4 as fp4fmt
        return fp4fmt.pack_mmfp4(*fp4fmt.quantize_codes(w, group_size))
    w = w.detach().contiguous()
    packed = torch.empty(w.shape[0], w.shape[1] // 8, dtype=torch.int32, device=w.device)
    scales = torch.empty(w.shape[0], w.shape[1] // group_size, dtype=torch.float16, device=w.device)
    K.mmb200.fp4_quantize_pack(w, packed, scales, group_size)
    return packed, scales


def hadamard(x, block: int = 128, out=None):
    """Orthonormal block Walsh-Hadamard transform along the last axis (bf16 on CUDA; any float dtype on CPU)."""
    if not _use_native(x) or x.dtype != torch.bfloat16:
        from ..quant.hadamard import fwht
        D = x.shape[-1]
        y = fwht(x.reshape(*x.shape[:-1], D // block, block)).reshape(x.shape)
        if out is not None:
            out.copy_(y)
            return out
        return y
    x = x.contiguous()
    if out is None:
        out = torch.empty_like(x)
    K.mmb200.hadamard(x, out, block)
    return out


def trellis_dequant(codes, scales, su, sv, out_f: int, in_f: int, bits: int, group_size: int, out=None):
    """bf16 ``[out, in]`` from the header-less trellis tile bit stream (``formats/trellis.py`` layout)."""
    if not _use_native(codes):
        from ..formats import trellis as tr
        blob = torch.cat([torch.tensor([bits], dtype=torch.uint8, device=codes.device), codes.reshape(-1)])
        w = tr.TrellisWeight(blob, scales, su, sv, (out_f, in_f)).dequantize(torch.bfloat16)
        if out is not None:
            out.copy_(w)
            return out
        return w
    if out is None:
        out = torch.empty(out_f, in_f, dtype=torch.bfloat16, device=codes.device)
    K.mmb200.trellis_dequant(codes, scales, su, sv, out, bits, group_size)
    return out


def trellis_desc_row(codes, scales, su, sv, out_f: int, in_f: int, bits: int, group_size: int):
    """One matrix descriptor (six int64) of the trellis kernels: codes, scales, su, sv, out | in << 32, bits | group << 32."""
    return [codes.data_ptr(), scales.data_ptr(), su.data_ptr(), sv.data_ptr(), out_f | (in_f << 32), bits | (group_size << 32)]


def trellis_gemm_ok(x, in_f: int, group_size: int) -> bool:
    """Whether the tensor-core trellis GEMM (codes decoded inside the main loop) takes this input."""
    return bool(_use_native(x) and x.dtype == torch.bfloat16 and in_f % 64 == 0 and group_size % 16 == 0 and not NO_TCGEN05)


def trellis_gemm(x, desc, N: int, Kin: int, *, act: int = 0, first: int = 0, stride: int = 1, tiles=None, token_tile: int = 0,
                 row_scale=None, out=None, out_rows=None):
    """``out = x @ W^T`` with trellis weights decoded in the tcgen05 GEMM's main loop (2..8 bits, mixed per matrix).
    ``desc``: device int64 ``[n_mats, 6]`` (:func:`trellis_desc_row`).  ``act=1``: matrices ``first`` (gate) and
    ``first + 1`` (up), SwiGLU in the epilogue, ``out [M, N / 2]``.  ``tiles = (tile_expert, tile_row0, tile_rows, n_tiles)``:
    grouped mode over rows sorted by expert (matrix ``expert * stride + first``).  ``out_rows`` (device int64 per row): the
    scatter epilogue of the expert-parallel return path (``out`` then only gives the row width)."""
    M = x.shape[0]
    if out is None:
        out = torch.empty(M, N // 2 if act else N, dtype=torch.bfloat16, device=x.device)
    te = tr0 = trw = nt = None
    if tiles is not None:
        te, tr0, trw, nt = tiles
    K.mmb200.trellis_gemm(x, desc, out, N, Kin, act, first, stride, te, tr0, trw, nt, token_tile, row_scale, out_rows, gemm_status(x.device))
    return out


def trellis_gemv(x, codes, scales, su, sv, out_f: int, bits: int, group_size: int, out=None):
    """``x [M, in] @ W^T`` for small M straight from the bit stream."""
    in_f = x.shape[1]
    if not _use_native(x) or group_size % 16 != 0:
        w = trellis_dequant(codes, scales, su, sv, out_f, in_f, bits, group_size)
        y = (x.to(torch.float32) @ w.to(torch.float32).t()).to(torch.bfloat16)
        if out is not None:
            out.copy_(y)
            return out
        return y
    if out is None:
        out = torch.empty(x.shape[0], out_f, dtype=torch.bfloat16, device=x.device)
    K.mmb200.trellis_gemv(x, codes, scales, su, sv, out, bits, group_size)
    return out


def codebook_gemv(x, codes, scales, zeros, lut, in_f: int, group_size: int, bits: int = 8, out=None):
    """``x [M <= 8, in] @ W^T`` with ``W = (lut[code] - zero) * scale``; ``codes uint8 [out, in * bits / 8]`` packed
    LSB-first (bits 2 / 4 / 8), ``scales`` / ``zeros`` fp16 ``[out, in / gs]``, ``lut`` fp32 [256]."""
    if not _use_native(x):
        w = ref.codebook_dequant(codes, scales, zeros, lut, in_f, group_size, bits)
        y = (x[:, :in_f].to(torch.float32) @ w.t()).to(torch.bfloat16)
        if out is not None:
            out.copy_(y)
            return out
        return y
    if out is None:
        out = torch.empty(x.shape[0], codes.shape[0], dtype=torch.bfloat16, device=x.device)
    K.mmb200.codebook_gemv(x, codes, scales, zeros, lut, out, in_f, group_size, bits)
    return out


def codebook_gemm_ok(x, in_f: int, group_size: int, bits: int) -> bool:
    """Whether the tensor-core codebook GEMM takes this problem (else: de-quantize and use the bf16 GEMM)."""
    return (_use_native(x) and not NO_TCGEN05 and x.dtype == torch.bfloat16 and bits in (2, 4, 8) and in_f % 64 == 0
            and group_size >= 32 and group_size & (group_size - 1) == 0 and in_f % group_size == 0)


def codebook_gemm(x, codes, scales, zeros, lut, in_f: int, group_size: int, bits: int = 8, out=None):
    """``x [M, in] @ W^T`` for any ``M`` with the codebook weights of :func:`codebook_gemv`, expanded inside the tcgen05 GEMM's
    main loop (no bf16 copy of the matrix exists)."""
    if not codebook_gemm_ok(x, in_f, group_size, bits):
        w = ref.codebook_dequant(codes, scales, zeros, lut, in_f, group_size, bits)
        y = (x[:, :in_f].to(torch.float32) @ w.t()).to(torch.bfloat16)
        if out is not None:
            out.copy_(y)
            return out
        return y
    if out is None:
        out = torch.empty(x.shape[0], codes.shape[0], dtype=torch.bfloat16, device=x.device)
    K.mmb200.codebook_gemm(x.contiguous(), codes, scales, zeros, lut, out, in_f, group_size, bits, gemm_status(x.device))
    return out


def sparse24_gemm(x, codes, meta, scales, in_f: int, group_size: int, out=None):
    """``x [M, in] @ W^T`` with 2:4 sparse FP4 weights (``layers.Sparse24Linear``): the kept values are scattered to their
    columns inside the tcgen05 GEMM's main loop.  Off the GPU: the product over the de-quantized dense matrix."""
    ok = (_use_native(x) and not NO_TCGEN05 and x.dtype == torch.bfloat16 and in_f % 64 == 0 and group_size >= 32
          and group_size & (group_size - 1) == 0 and in_f % group_size == 0)
    if not ok:
        w = ref.sparse24_dequant(codes, meta, scales, in_f, group_size)
        y = (x[:, :in_f].to(torch.float32) @ w.t()).to(torch.bfloat16)
        if out is not None:
            out.copy_(y)
            return out
        return y
    if out is None:
        out = torch.empty(x.shape[0], codes.shape[0], dtype=torch.bfloat16, device=x.device)
    K.mmb200.sparse24_gemm(x.contiguous(), codes, meta, scales, out, in_f, group_size, gemm_status(x.device))
    return out


def vision_preprocess(images, out_h: int, out_w: int, *, patch: int = 0, mean=(0.48145466, 0.4578275, 0.40821073),
                      std=(0.26862954, 0.26130258, 0.27577711)):
    """uint8 ``[B, H, W, 3]`` -> bf16 ``[B, 3, out_h, out_w]`` (``patch == 0``) or patches ``[B, n, 3 * patch^2]``."""
    B = images.shape[0]
    if not _use_native(images):
        return ref.vision_preprocess(images, out_h, out_w, patch, mean, std)
    shape = (B, 3, out_h, out_w) if patch == 0 else (B, (out_h // patch) * (out_w // patch), 3 * patch * patch)
    out = torch.empty(*shape, dtype=torch.bfloat16, device=images.device)
    K.mmb200.vision_preprocess(images.contiguous(), out, out_h, out_w, patch, [float(m) for m in mean], [float(s) for s in std])
    return out


RESAMPLE_MODES = {"bilinear": 0, "bicubic": 1, "nearest": 2}


def vision_preprocess_ex(images, out_h: int, out_w: int, *, crop=None, patch: int = 0, merge: int = 1, resample: str = "bilinear",
                         mean=(0.48145466, 0.4578275, 0.40821073), std=(0.26862954, 0.26130258, 0.27577711)):
    """General image preprocessing in one launch: ``crop = (y, x, h, w)`` source rectangle (None = whole image), resampling
    to ``out_h x out_w`` (bilinear / bicubic / nearest, half-pixel centres), normalisation, CHW pixels or ViT patches
    (``merge > 1``: patches ordered by merge x merge groups).  Parity: reference ``src/vision_preprocess.metal:214`` (bicubic),
    ``:761`` (centre crop), ``:1354`` (patch extraction)."""
    B, H, W, _ = images.shape
    crop = (0, 0, H, W) if crop is None else tuple(int(c) for c in crop)
    if not _use_native(images):
        return ref.vision_preprocess_ex(images, out_h, out_w, crop, patch, merge, resample, mean, std)
    shape = (B, 3, out_h, out_w) if patch == 0 else (B, (out_h // patch) * (out_w // patch), 3 * patch * patch)
    out = torch.empty(*shape, dtype=torch.bfloat16, device=images.device)
    K.mmb200.vision_preprocess_ex(images.contiguous(), out, list(crop), out_h, out_w, patch, merge, RESAMPLE_MODES[resample],
                                  [float(m) for m in mean], [float(s) for s in std])
    return out


def channel_stats(images):
    """Per-image, per-channel (mean, std) of ``pixel / 255`` for uint8 ``[B, H, W, 3]`` images: fp32 ``[B, 3, 2]``."""
    if not _use_native(images):
        v = images.to(torch.float32) / 255.0
        return torch.stack([v.mean((1, 2)), v.std((1, 2), unbiased=False)], -1)
    out = torch.empty(images.shape[0], 3, 2, dtype=torch.float32, device=images.device)
    K.mmb200.channel_stats(images.contiguous(), out)
    return out


def spec_verify(p_target, p_draft, draft, u, u_resample):
    """Rejection-sampling verification of ``K`` draft tokens per sequence.  Returns ``(tokens int64 [B, K + 1]``
    padded with -1, ``accepted int32 [B])``; ``tokens[b, :accepted[b] + 1]`` are the tokens to commit."""
    if not _use_native(p_target):
        return ref.spec_verify(p_target, p_draft, draft, u, u_resample)
    B, K1, V = p_target.shape
    toks = torch.empty(B, K1, dtype=torch.int64, device=p_target.device)
    acc = torch.empty(B, dtype=torch.int32, device=p_target.device)
    K.mmb200.spec_verify(p_target.contiguous(), p_draft.contiguous(), draft.contiguous(), u.contiguous(), u_resample.contiguous(), toks, acc)
    return toks, acc


PREFILL_ATTN_DIMS = (64, 128, 256)


FMHA_TCGEN05 = os.environ.get("MMB200_FMHA", "1") != "0"      # single-sequence causal prompts take the tcgen05 attention kernel
FMHA_MIN_T = 256


def fmha_ok(t: int, n: int, D: int, Dv: int, device) -> bool:
    """True when a single causal sequence of ``t`` queries over ``n`` keys takes the tcgen05 attention kernel."""
    return bool(FMHA_TCGEN05 and not NO_TCGEN05 and D == Dv and D in (128, 256) and t >= FMHA_MIN_T and n >= t
                and torch.device(device).type == "cuda" and native_available() and not _FORCE_REF)


def fmha_prefill(q, k, v, out, scale, vt=None, window=0):
    """Causal attention of ONE sequence on the tcgen05 kernel (``csrc/attention_fmha_sm100.cu``): ``q [t, Hq, D]`` are the last
    ``t`` positions of the keys ``k, v [n, Hk, D]``; ``D`` 128 or 256.  With ``window > 0`` a query sees only the last
    ``window`` keys up to its own position, and key tiles in front of a query tile's window are skipped.  The kernel takes V transposed per head, ``vt [Hk, D,
    n_pad]`` with ``n_pad % 8 == 0`` and zeros behind column ``n`` (the B operand of its P V MMA is K-major like every other
    operand); callers that can produce it directly (a GEMM with swapped operands) pass ``vt``, else it is built here with
    one strided copy of ``v``."""
    assert native_available(), "the tcgen05 attention kernel needs the CUDA extension"
    n, Hk, D = k.shape
    if vt is None:
        n_pad = (n + 7) // 8 * 8
        vt = torch.empty(Hk, D, n_pad, dtype=torch.bfloat16, device=q.device)
        vt[:, :, :n].copy_(v.permute(1, 2, 0))
        if n_pad > n:
            vt[:, :, n:].zero_()
    K.mmb200.fmha_prefill(q, k, vt, out, n, float(scale), gemm_status(q.device), int(window or 0))
    return out


def prefill_attention(q, k, v, cu_q, *, cu_k=None, block_tables=None, ctx_lens=None, block_size=16, max_q=None, scale=None, window=0,
                      causal=True, out=None, q_lens_host=None, k_lens_host=None, sinks=0, tree_mask=None, block_mask=None):
    """Variable-length prefill attention.  ``q [T, Hq, D]``; contiguous keys ``k, v [N, Hk, D]`` with ``cu_k``, or paged
    pools ``[slots, Hk, D]`` with ``block_tables`` / ``ctx_lens``.  The queries of a sequence are the last positions of
    its keys.  ``cu_q`` / ``cu_k``: int32 device tensors ``[B + 1]``.

    Mask modes (combined by AND): ``causal``; ``window`` (+ ``sinks`` always-visible first keys); ``tree_mask`` uint8
    ``[T, >= max_q]`` - query row i sees the j-th of its sequence's last ``q_len`` keys iff ``tree_mask[i, j]`` (earlier keys
    stay visible; pass ``causal=False`` for a token tree); ``block_mask`` uint8 ``[1 | Hq, ceil(max_q / 128), n_kblocks]`` -
    128-query x 64-key blocks with a zero byte are skipped."""
    T, Hq, D = q.shape
    scale = scale if scale is not None else D ** -0.5
    if out is None:
        out = torch.empty(T, Hq, D, dtype=torch.bfloat16, device=q.device)
    if isinstance(k, FP8KV):
        # prompt pass over a quantized cache: the sequences' rows are de-quantized into contiguous bf16 keys / values once
        # (one gather launch per pool) and the kernel runs in its contiguous mode
        lens = ctx_lens.to(torch.int64)
        cu_k = torch.zeros(lens.numel() + 1, dtype=torch.int32, device=q.device)
        cu_k[1:] = torch.cumsum(lens, 0)
        total, mx = int(cu_k[-1]), int(lens.max())
        k, v = (kv_fp8_rows(pl, block_tables, ctx_lens, cu_k, total, mx, block_size) for pl in (k, v))
        block_tables = ctx_lens = None
    if max_q is None and (block_mask is not None or (_use_native(q) and D in PREFILL_ATTN_DIMS)):
        max_q = int((cu_q[1:] - cu_q[:-1]).max())
    if (FMHA_TCGEN05 and _use_native(q) and not NO_TCGEN05 and D in (128, 256) and q.dtype == torch.bfloat16 and cu_k is not None
            and cu_q.numel() == 2 and causal and not sinks and tree_mask is None and block_mask is None
            and T >= FMHA_MIN_T and k.shape[-1] == D and v.shape[-1] == D and k.shape[0] >= T and q.stride(2) == 1
            and k.stride(2) == 1 and out.stride(2) == 1 and k.stride(1) <= k.stride(0) and q.stride(1) <= q.stride(0)):
        return fmha_prefill(q, k, v, out, scale, window=window)
    if _use_native(q) and D in PREFILL_ATTN_DIMS and q.dtype == torch.bfloat16 and k.shape[-1] == D and v.shape[-1] == D:
        K.mmb200.prefill_attention(q, k, v, out, cu_q, cu_k, block_tables, ctx_lens, block_size, max_q, scale, window, causal,
                                   int(sinks), tree_mask, block_mask)
        return out
    return ref.prefill_attention(q, k, v, cu_q, cu_k, block_tables, ctx_lens, block_size, scale, window, causal, out,
                                 sinks=sinks, tree_mask=tree_mask, block_mask=block_mask)


if os.environ.get("MMB200_TUNING_FILE"):      # a table written by `metal-marlin autotune` replaces the built-in thresholds
    from ..autotune import load_config as _load_tuning
    _load_tuning()


def __getattr__(name: str):
    # operation objects of the reference's ``ops`` package (GEMM classes, int8 packer, quantized linear module)
    if name in ("GemmFp4", "GemmInt8", "pack_int8_weights", "unpack_int8_weights"):
        from .. import compat_api
        return getattr(compat_api, name)
    if name == "MetalQuantizedLinear":
        from ..hf import QuantizedLinearModule
        return QuantizedLinearModule
    raise AttributeError(name)
