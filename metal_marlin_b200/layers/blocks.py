"""Stand-alone layer objects over FP4 weights: a mixture-of-experts layer (router, routed experts, shared experts), a
multi-head-latent-attention layer with its latent cache, and a linear layer whose format follows a precision policy.
Inside the engine these computations are methods of the shared decoder (``models/transformer.py``) over the paged cache;
the objects here serve code that builds a model layer by layer, as the reference's ``layers`` package does.

Parity: reference ``metal_marlin/layers/mmfp4_moe.py`` (``MMFP4MoE`` ``:352``: router -> softmax -> top-k -> renormalise, per-expert
SwiGLU, shared expert always added), ``layers/mmfp4_mla.py`` (``MMFP4MLA`` ``:149``: ``q_a -> norm -> q_b``, ``kv_a -> [c_kv | k_rope]``,
``kv_a_layernorm``, ``kv_b -> [k_nope | v]``, decoupled RoPE, ``o_proj``, latent KV cache), ``layers/mmfp4_mtp_head.py``
(``MMFP4MTPHead``, ``verify_kernel``) and ``mixed_precision`` linear selection.
"""
from __future__ import annotations

from typing import Dict, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

from .. import ops
from ..ops.weights import FP4ExpertBank
from .linear import MMFP4Linear, QuantizedLinear
from .lora import LoRAMixin


class MMFP4MoE:
    """``y = sum_k w_k expert_k(x) + shared(x)`` with FP4 expert banks on the engine's MoE kernels (per-slot streaming,
    expert-sorted streaming or grouped tcgen05 GEMM by token count)."""

    def __init__(self, router_weight: torch.Tensor, gate_up: FP4ExpertBank, down: FP4ExpertBank, top_k: int, num_shared: int = 0,
                 scoring: str = "softmax", renormalize: bool = True, routed_scale: float = 1.0, correction_bias: Optional[torch.Tensor] = None,
                 n_group: int = 1, topk_group: int = 1):
        self.router_weight, self.gate_up, self.down = router_weight.to(torch.bfloat16), gate_up, down
        self.top_k, self.num_shared = top_k, num_shared
        self.num_experts = gate_up.num_experts - num_shared
        self.scoring = {"softmax": 0, "sigmoid": 1}[scoring]
        self.renormalize, self.routed_scale, self.correction_bias = renormalize, routed_scale, correction_bias
        self.n_group, self.topk_group = n_group, topk_group

    @classmethod
    def from_float(cls, router_weight: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor, top_k: int,
                   shared: Optional[Tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = None, group_size: int = 128, device=None, **kw) -> "MMFP4MoE":
        """``gate, up [E, I, H]``, ``down [E, H, I]``; ``shared``: ``(gate [S, I, H], up [S, I, H], down [S, H, I])`` appended
        after the routed experts."""
        dev = device or gate.device
        gu = torch.cat([gate, up], 1)
        dn = down
        ns = 0
        if shared is not None:
            ns = shared[0].shape[0]
            gu = torch.cat([gu, torch.cat([shared[0], shared[1]], 1)], 0)
            dn = torch.cat([dn, shared[2]], 0)
        bank = lambda w: FP4ExpertBank.from_float(w.float().to(dev), group_size)
        return cls(router_weight.to(dev), bank(gu), bank(dn), top_k, ns, **kw)

    def route(self, x: torch.Tensor):
        return ops.moe_router(x, self.router_weight, bias=self.correction_bias, topk=self.top_k, scoring=self.scoring,
                              renorm=self.renormalize, routed_scale=self.routed_scale, n_group=self.n_group, topk_group=self.topk_group)

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        shape = x.shape
        x2 = x.reshape(-1, shape[-1]).to(torch.bfloat16).contiguous()
        ids, weights = self.route(x2)
        y = ops.moe_forward(x2, self.gate_up, self.down, ids, weights, n_shared=self.num_shared, shared_base=self.num_experts)
        return y.view(shape).to(x.dtype)

    forward = __call__


MMFP4FusedMoE = MMFP4MoE


def _rms(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()).to(x.dtype)


class MMFP4MLA:
    """Multi-head latent attention layer: low-rank query path, compressed key / value latent with a decoupled rotary slice,
    causal attention, output projection.  The cache stores the latent rows (``kv_lora_rank + rope_dim`` values per token)."""

    def __init__(self, weights: Dict[str, object], num_heads: int, qk_nope_head_dim: int, qk_rope_head_dim: int, v_head_dim: int,
                 kv_lora_rank: int, rope_theta: float = 10000.0, eps: float = 1e-6, interleaved: bool = True, scale: Optional[float] = None):
        self.w, self.H = weights, num_heads
        self.dn, self.dr, self.dv, self.R = qk_nope_head_dim, qk_rope_head_dim, v_head_dim, kv_lora_rank
        self.eps, self.interleaved = eps, interleaved
        self.scale = scale if scale is not None else (qk_nope_head_dim + qk_rope_head_dim) ** -0.5
        from ..rope import rope_inv_freq
        self.inv_freq, self.mscale = rope_inv_freq(qk_rope_head_dim, rope_theta)

    @classmethod
    def from_float(cls, hidden: int, num_heads: int, q_lora_rank: int, kv_lora_rank: int, qk_nope_head_dim: int, qk_rope_head_dim: int,
                   v_head_dim: int, state: Optional[Dict[str, torch.Tensor]] = None, group_size: int = 64, seed: int = 0, device="cpu", **kw):
        """``state``: float tensors ``q_a_proj``, ``q_a_layernorm``, ``q_b_proj``, ``kv_a_proj_with_mqa``, ``kv_a_layernorm``,
        ``kv_b_proj``, ``o_proj`` (random when absent)."""
        g = torch.Generator().manual_seed(seed)
        rn = lambda *s: torch.randn(*s, generator=g) * 0.05
        H, dn, dr, dv = num_heads, qk_nope_head_dim, qk_rope_head_dim, v_head_dim
        st = dict(state or {})
        st.setdefault("q_a_proj", rn(q_lora_rank, hidden))
        st.setdefault("q_a_layernorm", torch.ones(q_lora_rank))
        st.setdefault("q_b_proj", rn(H * (dn + dr), q_lora_rank))
        st.setdefault("kv_a_proj_with_mqa", rn(kv_lora_rank + dr, hidden))
        st.setdefault("kv_a_layernorm", torch.ones(kv_lora_rank))
        st.setdefault("kv_b_proj", rn(H * (dn + dv), kv_lora_rank))
        st.setdefault("o_proj", rn(hidden, H * dv))
        lin = lambda n: MMFP4Linear.from_float(st[n].float(), group_size, device=device)
        w = {"q_a": lin("q_a_proj"), "q_a_norm": st["q_a_layernorm"].to(device), "q_b": lin("q_b_proj"), "kv_a": lin("kv_a_proj_with_mqa"),
             "kv_a_norm": st["kv_a_layernorm"].to(device), "kv_b": lin("kv_b_proj"), "o": lin("o_proj")}
        return cls(w, H, dn, dr, dv, kv_lora_rank, **kw)

    def new_cache(self, batch: int = 1, max_seq_len: int = 4096, dtype: str = "bf16", device="cpu"):
        from ..kv.contiguous import MLAKVCache
        return MLAKVCache(1, self.R, self.dr, batch, max_seq_len, dtype, device)

    def _rope(self, x: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        from ..rope import apply_rope
        B, T = x.shape[:2]
        y = apply_rope(x.reshape(B * T, *x.shape[2:]), positions.reshape(-1), self.inv_freq, interleaved=self.interleaved, mscale=self.mscale)
        return y.reshape(x.shape)

    def __call__(self, x: torch.Tensor, positions: Optional[torch.Tensor] = None, cache=None, layer: int = 0) -> torch.Tensor:
        """``x [B, T, hidden]``; with ``cache`` (``new_cache()``) the layer attends over everything cached so far plus ``x``."""
        w, B, T = self.w, x.shape[0], x.shape[1]
        H, dn, dr, dv, R = self.H, self.dn, self.dr, self.dv, self.R
        past = cache.seq_len if cache is not None else 0
        if positions is None:
            positions = torch.arange(past, past + T, device=x.device).expand(B, T)
        q = w["q_b"](_rms(w["q_a"](x), w["q_a_norm"], self.eps)).view(B, T, H, dn + dr)
        q_nope, q_rope = q[..., :dn], self._rope(q[..., dn:], positions)
        kva = w["kv_a"](x)
        c = _rms(kva[..., :R], w["kv_a_norm"], self.eps)
        k_rope = self._rope(kva[..., R:].unsqueeze(2), positions).squeeze(2)
        latent = torch.cat([c, k_rope], -1)
        if cache is not None:
            latent = cache.update_compressed(layer, latent, dtype=latent.dtype)
        S = latent.shape[1]
        kvb = w["kv_b"](latent[..., :R]).view(B, S, H, dn + dv)
        k = torch.cat([kvb[..., :dn], latent[..., R:].unsqueeze(2).expand(B, S, H, dr)], -1)
        qq = torch.cat([q_nope, q_rope], -1)
        mask = torch.arange(S, device=x.device).view(1, S) <= torch.arange(S - T, S, device=x.device).view(T, 1)
        o = F.scaled_dot_product_attention(qq.transpose(1, 2).float(), k.transpose(1, 2).float(), kvb[..., dn:].transpose(1, 2).float(),
                                           attn_mask=mask, scale=self.scale)
        return w["o"](o.transpose(1, 2).reshape(B, T, H * dv).to(x.dtype))

    forward = __call__


class MixedPrecisionLinear(LoRAMixin):
    """A linear layer whose storage follows a precision policy: ``fp4`` -> :class:`MMFP4Linear`, other quantized formats ->
    :class:`QuantizedLinear`, 16-bit formats stay a plain matrix."""

    def __init__(self, weight: torch.Tensor, precision="fp4", group_size: int = 128, bias: Optional[torch.Tensor] = None, device=None):
        fmt = getattr(precision, "value", precision)
        self.format = fmt
        dev = device or weight.device
        if fmt == "fp4":
            self.inner = MMFP4Linear.from_float(weight.float(), group_size, bias=None if bias is None else bias.to(dev, torch.bfloat16), device=dev)
        elif fmt in ("bf16", "fp16", "keep"):
            self.inner = None
            self.weight = weight.to(dev, torch.bfloat16 if fmt != "fp16" else torch.float16)
            self.bias = None if bias is None else bias.to(dev)
        else:
            self.inner = QuantizedLinear.from_float(weight.float(), fmt, group_size, bias=bias, device=dev)
        self.out_features, self.in_features = weight.shape

    @classmethod
    def for_tensor(cls, name: str, weight: torch.Tensor, preset: str = "dense", **kw) -> "MixedPrecisionLinear":
        from ..quant.mixed_precision import policy_for
        pol = policy_for(name, preset)
        return cls(weight, pol.fmt, pol.group_size or 128, **kw)

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        if self.inner is not None:
            return self.inner(x).to(x.dtype)
        return F.linear(x.to(self.weight.dtype), self.weight, None if self.bias is None else self.bias.to(self.weight.dtype)).to(x.dtype)


def verify_kernel(p_target: torch.Tensor, p_draft: torch.Tensor, draft_tokens: torch.Tensor, uniform: Optional[torch.Tensor] = None,
                  uniform_resample: Optional[torch.Tensor] = None, generator: Optional[torch.Generator] = None):
    """Vectorised rejection-sampling verification of ``K`` drafted tokens per sequence: ``p_target [B, K + 1, V]``, ``p_draft [B, K, V]``,
    ``draft_tokens [B, K]`` -> ``(tokens [B, K + 1] padded with -1, accepted [B])`` (the verification kernel on a GPU)."""
    B, K1, _V = p_target.shape
    dev = p_target.device
    u = uniform if uniform is not None else torch.rand(B, K1 - 1, generator=generator).to(dev)
    ur = uniform_resample if uniform_resample is not None else torch.rand(B, generator=generator).to(dev)
    return ops.spec_verify(p_target.float(), p_draft.float(), draft_tokens.to(torch.int64), u.float(), ur.float())
