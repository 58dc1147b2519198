"""Block-level classes of the alternative architectures: RWKV-6 time mixing / channel mixing / block with its layer state,
a differential-attention module, and a hybrid stack builder that assembles attention, Mamba and RWKV blocks from a layout
and carries every block's state between calls.

Parity: reference ``metal_marlin/architectures/rwkv.py`` (``RWKVTimeMixing``, ``RWKVChannelMixing``, ``RWKVBlock``, ``RWKVLayerState``,
``rwkv_wkv_batched``, ``rwkv_wkv_single_token``), ``architectures/diff_transformer.py`` (``DifferentialAttentionConfig``,
``DifferentialAttention``, ``parse_diff_transformer_config``), ``architectures/hybrid.py`` (``HybridLayerType``, ``HybridLayerConfig``,
``HybridArchitectureConfig``, ``HybridBlock``, ``HybridModel``, ``HybridModelBuilder``, ``build_hybrid_config``, ``LayerState``,
``StateType``) and ``architectures/mamba.py`` (``MarlinMambaBlock``, ``MambaState``, ``MambaLayerConfig``, ``SelectiveScanConfig``).
The recurrences run on the scan kernels of ``csrc/recurrent_scan.cu`` when the tensors are on a GPU.
"""
from __future__ import annotations

import enum
import math
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Protocol, Sequence, Tuple

import torch
import torch.nn.functional as F

from .mamba import MambaBlock, MambaConfig
from .rwkv import wkv6


# ------------------------------------------------------------------------------------------------ RWKV-6
def rwkv_wkv_batched(r, k, v, w, u, state: Optional[torch.Tensor] = None):
    """``r, k [B, T, H, dk]``, ``v [B, T, H, dv]``, decay ``w [B, T, H, dk]`` in (0, 1), bonus ``u [H, dk]`` -> ``(out [B, T, H, dv],
    state [B, H, dk, dv])``."""
    return wkv6(r, k, v, w.contiguous(), u, state)


def rwkv_wkv_single_token(r, k, v, w, u, state: torch.Tensor):
    """One token: ``r, k, w [B, H, dk]``, ``v [B, H, dv]`` with the running ``state``; returns ``(out [B, H, dv], new state)``."""
    o, s = wkv6(r[:, None], k[:, None], v[:, None], w[:, None].contiguous(), u, state)
    return o[:, 0], s


@dataclass
class RWKVLayerState:
    time_shift: Optional[torch.Tensor] = None        # [B, d] last input of the time-mixing branch
    channel_shift: Optional[torch.Tensor] = None     # [B, d] last input of the channel-mixing branch
    wkv: Optional[torch.Tensor] = None               # [B, H, dk, dv]


def _shift(x: torch.Tensor, prev: Optional[torch.Tensor]) -> torch.Tensor:
    """Token shift: every position sees its predecessor (the carried row, or zeros, for the first one)."""
    first = prev[:, None] if prev is not None else torch.zeros_like(x[:, :1])
    return torch.cat([first, x[:, :-1]], 1)


class RWKVTimeMixing:
    """RWKV-6 time mixing: data-dependent token-shift interpolation (a low-rank ``tanh`` adapter gives five mixing vectors),
    receptance / key / value / gate projections, a low-rank data-dependent decay, the WKV recurrence, per-head group
    normalisation and the gated output projection."""

    def __init__(self, d_model: int, n_heads: int, weights: Dict[str, torch.Tensor]):
        self.d, self.H, self.hd, self.w = d_model, n_heads, d_model // n_heads, weights

    @classmethod
    def random(cls, d_model: int, n_heads: int, lora: int = 32, decay_lora: int = 64, seed: int = 0, device="cpu") -> "RWKVTimeMixing":
        g = torch.Generator().manual_seed(seed)
        rn = lambda *s, std=0.05: (torch.randn(*s, generator=g) * std).to(device)
        d = d_model
        w = {"maa_x": rn(d), "maa": rn(5, d), "maa_w1": rn(d, 5 * lora), "maa_w2": rn(5, lora, d), "decay": rn(d) - 4.0,
             "decay_w1": rn(d, decay_lora), "decay_w2": rn(decay_lora, d), "bonus": rn(n_heads, d // n_heads),
             "wr": rn(d, d), "wk": rn(d, d), "wv": rn(d, d), "wg": rn(d, d), "wo": rn(d, d),
             "ln_w": torch.ones(d, device=device), "ln_b": torch.zeros(d, device=device)}
        return cls(d_model, n_heads, w)

    def __call__(self, x: torch.Tensor, state: Optional[RWKVLayerState] = None) -> Tuple[torch.Tensor, RWKVLayerState]:
        w, B, T = self.w, x.shape[0], x.shape[1]
        st = state or RWKVLayerState()
        xf = x.float()
        dx = _shift(xf, st.time_shift) - xf
        xxx = xf + dx * w["maa_x"]
        mix = torch.tanh(xxx @ w["maa_w1"]).view(B, T, 5, -1).permute(2, 0, 1, 3)              # [5, B, T, lora]
        mix = torch.einsum("fbtl,fld->fbtd", mix, w["maa_w2"]) + w["maa"][:, None, None, :]
        xw, xk, xv, xr, xg = (xf + dx * mix[i] for i in range(5))
        r = (xr @ w["wr"].t()).view(B, T, self.H, self.hd)
        k = (xk @ w["wk"].t()).view(B, T, self.H, self.hd)
        v = (xv @ w["wv"].t()).view(B, T, self.H, self.hd)
        gate = F.silu(xg @ w["wg"].t())
        decay = w["decay"] + torch.tanh(xw @ w["decay_w1"]) @ w["decay_w2"]
        wdec = torch.exp(-torch.exp(decay)).view(B, T, self.H, self.hd)
        o, s = rwkv_wkv_batched(r, k, v, wdec, w["bonus"], st.wkv)
        o = F.group_norm(o.float().reshape(B * T, self.d), self.H, w["ln_w"], w["ln_b"], eps=64e-5).view(B, T, self.d)
        y = (o * gate) @ w["wo"].t()
        return y.to(x.dtype), RWKVLayerState(xf[:, -1].clone(), st.channel_shift, s)


class RWKVChannelMixing:
    """``sigmoid(W_r x_r) * W_v relu(W_k x_k)^2`` with token-shift interpolation of the inputs."""

    def __init__(self, d_model: int, d_ffn: int, weights: Dict[str, torch.Tensor]):
        self.d, self.f, self.w = d_model, d_ffn, weights

    @classmethod
    def random(cls, d_model: int, d_ffn: Optional[int] = None, seed: int = 0, device="cpu") -> "RWKVChannelMixing":
        g = torch.Generator().manual_seed(seed)
        f = d_ffn or int(3.5 * d_model) // 32 * 32
        rn = lambda *s: (torch.randn(*s, generator=g) * 0.05).to(device)
        return cls(d_model, f, {"maa_k": rn(d_model), "maa_r": rn(d_model), "wk": rn(f, d_model), "wv": rn(d_model, f), "wr": rn(d_model, d_model)})

    def __call__(self, x: torch.Tensor, state: Optional[RWKVLayerState] = None) -> Tuple[torch.Tensor, RWKVLayerState]:
        w = self.w
        st = state or RWKVLayerState()
        xf = x.float()
        dx = _shift(xf, st.channel_shift) - xf
        xk, xr = xf + dx * w["maa_k"], xf + dx * w["maa_r"]
        kk = torch.relu(xk @ w["wk"].t()) ** 2
        y = torch.sigmoid(xr @ w["wr"].t()) * (kk @ w["wv"].t())
        return y.to(x.dtype), RWKVLayerState(st.time_shift, xf[:, -1].clone(), st.wkv)


class RWKVBlock:
    """``x + TimeMix(LN1 x)`` then ``x + ChannelMix(LN2 x)``; the state is carried across calls, so a prompt pass followed by
    single-token calls equals one pass over the whole sequence."""

    def __init__(self, time_mix: RWKVTimeMixing, channel_mix: RWKVChannelMixing, ln1=None, ln2=None):
        d = time_mix.d
        dev = time_mix.w["wr"].device
        one = lambda: (torch.ones(d, device=dev), torch.zeros(d, device=dev))
        self.tm, self.cm, self.ln1, self.ln2 = time_mix, channel_mix, ln1 or one(), ln2 or one()

    @classmethod
    def random(cls, d_model: int, n_heads: int, seed: int = 0, device="cpu") -> "RWKVBlock":
        return cls(RWKVTimeMixing.random(d_model, n_heads, seed=seed, device=device), RWKVChannelMixing.random(d_model, seed=seed + 1, device=device))

    def __call__(self, x: torch.Tensor, state: Optional[RWKVLayerState] = None) -> Tuple[torch.Tensor, RWKVLayerState]:
        d = x.shape[-1]
        h, st = self.tm(F.layer_norm(x.float(), (d,), *self.ln1), state)
        x = x + h.to(x.dtype)
        h, st = self.cm(F.layer_norm(x.float(), (d,), *self.ln2), st)
        return x + h.to(x.dtype), st


# ------------------------------------------------------------------------------------------------ Mamba names
MarlinMambaBlock = MambaBlock
MambaLayerConfig = MambaConfig
SelectiveScanConfig = MambaConfig


@dataclass
class MambaState:
    conv: torch.Tensor           # [B, d_inner, d_conv - 1]
    ssm: torch.Tensor            # [B, d_inner, d_state]

    def as_tuple(self):
        return self.conv, self.ssm


# ------------------------------------------------------------------------------------------------ differential attention
@dataclass
class DifferentialAttentionConfig:
    hidden_size: int = 512
    num_heads: int = 8                # each head is a pair of half-width query / key heads
    num_kv_heads: Optional[int] = None
    layer_idx: int = 0
    causal: bool = True

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_heads // 2

    @property
    def lambda_init(self) -> float:
        return 0.8 - 0.6 * math.exp(-0.3 * self.layer_idx)


def parse_diff_transformer_config(config: Dict[str, Any], layer_idx: int = 0) -> DifferentialAttentionConfig:
    return DifferentialAttentionConfig(int(config["hidden_size"]), int(config["num_attention_heads"]),
                                       config.get("num_key_value_heads"), layer_idx, bool(config.get("causal", True)))


class DifferentialAttention:
    """Differential attention layer: two soft-max maps from paired half-width heads are subtracted with a learned
    ``lambda`` (``exp(lq1 . lk1) - exp(lq2 . lk2) + lambda_init``), applied to double-width values, normalised per head."""

    def __init__(self, config: DifferentialAttentionConfig, weights: Dict[str, torch.Tensor]):
        self.cfg, self.w = config, weights

    @classmethod
    def random(cls, config: DifferentialAttentionConfig, seed: int = 0, device="cpu") -> "DifferentialAttention":
        g = torch.Generator().manual_seed(seed)
        d, hd = config.hidden_size, config.head_dim
        rn = lambda *s: (torch.randn(*s, generator=g) * 0.05).to(device)
        return cls(config, {"wq": rn(d, d), "wk": rn(d, d), "wv": rn(d, d), "wo": rn(d, d), "lq1": rn(hd), "lk1": rn(hd), "lq2": rn(hd),
                            "lk2": rn(hd), "subln": torch.ones(2 * hd, device=device)})

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        from ..attention import differential_attention
        c, w = self.cfg, self.w
        B, T, d = x.shape
        H, hd = c.num_heads, c.head_dim
        q = (x.float() @ w["wq"].t()).view(B, T, 2 * H, hd).transpose(1, 2)
        k = (x.float() @ w["wk"].t()).view(B, T, 2 * H, hd).transpose(1, 2)
        v = (x.float() @ w["wv"].t()).view(B, T, H, 2 * hd).transpose(1, 2)
        lam = float(torch.exp((w["lq1"] * w["lk1"]).sum()) - torch.exp((w["lq2"] * w["lk2"]).sum())) + c.lambda_init
        o = differential_attention(q[:, 0::2], k[:, 0::2], q[:, 1::2], k[:, 1::2], v, lam, c.lambda_init, w["subln"], causal=c.causal)
        return (o.transpose(1, 2).reshape(B, T, d).float() @ w["wo"].t()).to(x.dtype)


DifferentialMarlinAttention = DifferentialAttention


# ------------------------------------------------------------------------------------------------ hybrid stacks
class HybridLayerType(enum.Enum):
    ATTENTION = "attention"
    MAMBA = "mamba"
    RWKV = "rwkv"
    DIFF_ATTENTION = "diff_attention"


class StateType(enum.Enum):
    NONE = "none"
    KV_CACHE = "kv_cache"
    RECURRENT = "recurrent"


@dataclass
class AttentionLayerConfig:
    num_heads: int = 8
    num_kv_heads: Optional[int] = None
    differential: bool = False


@dataclass
class HybridLayerConfig:
    layer_type: HybridLayerType
    attention: Optional[AttentionLayerConfig] = None
    mamba: Optional[MambaConfig] = None
    rwkv_heads: int = 8


@dataclass
class HybridArchitectureConfig:
    hidden_size: int
    layers: List[HybridLayerConfig]
    name: str = "hybrid"

    @property
    def num_layers(self) -> int:
        return len(self.layers)


def build_hybrid_config(kind: str, hidden_size: int, num_layers: int, num_heads: int = 8, **kw) -> HybridArchitectureConfig:
    """``jamba`` (one attention layer per ``attn_period`` Mamba layers), ``zamba`` (attention every ``shared_every``),
    ``rwkv`` (all RWKV), ``mamba`` (all Mamba), ``attention``."""
    from .hybrid import jamba_layout, zamba_layout
    att = lambda: HybridLayerConfig(HybridLayerType.ATTENTION, attention=AttentionLayerConfig(num_heads))
    mam = lambda: HybridLayerConfig(HybridLayerType.MAMBA, mamba=MambaConfig(d_model=hidden_size))
    if kind == "jamba":
        specs = jamba_layout(num_layers, kw.get("attn_period", 8), kw.get("attn_offset", 4))
        layers = [att() if s.mixer == "attention" else mam() for s in specs]
    elif kind == "zamba":
        layers = [att() if s.mixer == "shared_attention" else mam() for s in zamba_layout(num_layers, kw.get("shared_every", 6))]
    elif kind == "rwkv":
        layers = [HybridLayerConfig(HybridLayerType.RWKV, rwkv_heads=num_heads) for _ in range(num_layers)]
    elif kind == "mamba":
        layers = [mam() for _ in range(num_layers)]
    elif kind == "attention":
        layers = [att() for _ in range(num_layers)]
    else:
        raise ValueError(kind)
    return HybridArchitectureConfig(hidden_size, layers, kind)


@dataclass
class LayerState:
    kind: StateType = StateType.NONE
    value: Any = None


class LayerProtocol(Protocol):
    def __call__(self, x: torch.Tensor, state: Optional[LayerState]) -> Tuple[torch.Tensor, LayerState]: ...


class _AttentionMixer:
    """Plain multi-head causal attention that keeps its keys and values as the layer state."""

    def __init__(self, d: int, cfg: AttentionLayerConfig, seed: int, device):
        g = torch.Generator().manual_seed(seed)
        self.H, self.d = cfg.num_heads, d
        self.w = {n: (torch.randn(d, d, generator=g) * 0.05).to(device) for n in ("q", "k", "v", "o")}

    def __call__(self, x, state):
        B, T, d = x.shape
        hd = d // self.H
        q, k, v = ((x.float() @ self.w[n].t()).view(B, T, self.H, hd).transpose(1, 2) for n in ("q", "k", "v"))
        if state is not None and state.value is not None:
            k, v = torch.cat([state.value[0], k], 2), torch.cat([state.value[1], v], 2)
        n = k.shape[2]
        mask = torch.arange(n, device=x.device).view(1, n) <= torch.arange(n - T, n, device=x.device).view(T, 1)
        o = F.scaled_dot_product_attention(q, k, v, attn_mask=mask)
        return (o.transpose(1, 2).reshape(B, T, d) @ self.w["o"].t()).to(x.dtype), LayerState(StateType.KV_CACHE, (k, v))


class HybridBlock:
    """Pre-norm residual block around one mixer of the layer's type."""

    def __init__(self, hidden_size: int, cfg: HybridLayerConfig, seed: int = 0, device="cpu"):
        self.cfg, self.d = cfg, hidden_size
        t = cfg.layer_type
        if t is HybridLayerType.ATTENTION:
            self.mixer = _AttentionMixer(hidden_size, cfg.attention or AttentionLayerConfig(), seed, device)
        elif t is HybridLayerType.DIFF_ATTENTION:
            self.mixer = DifferentialAttention.random(DifferentialAttentionConfig(hidden_size, (cfg.attention or AttentionLayerConfig()).num_heads),
                                                      seed, device)
        elif t is HybridLayerType.MAMBA:
            self.mixer = MambaBlock.random(cfg.mamba or MambaConfig(d_model=hidden_size), seed, device)
        else:
            self.mixer = RWKVBlock.random(hidden_size, cfg.rwkv_heads, seed, device)

    def __call__(self, x: torch.Tensor, state: Optional[LayerState] = None) -> Tuple[torch.Tensor, LayerState]:
        t = self.cfg.layer_type
        if t is HybridLayerType.RWKV:                              # the RWKV block has its own norms and residuals
            y, st = self.mixer(x, None if state is None else state.value)
            return y, LayerState(StateType.RECURRENT, st)
        h = F.layer_norm(x.float(), (self.d,)).to(x.dtype)
        if t is HybridLayerType.MAMBA:
            y, st = self.mixer.forward(h, None if state is None else state.value)
            return x + y, LayerState(StateType.RECURRENT, st)
        if t is HybridLayerType.DIFF_ATTENTION:
            return x + self.mixer(h), LayerState(StateType.NONE)
        y, st = self.mixer(h, state)
        return x + y, st


class HybridModel:
    """A stack of hybrid blocks: ``forward(x [B, T, d], states) -> (y, states)``; feeding a sequence in pieces with the
    returned states equals feeding it at once."""

    def __init__(self, config: HybridArchitectureConfig, blocks: Sequence[HybridBlock]):
        self.config, self.blocks = config, list(blocks)

    def forward(self, x: torch.Tensor, states: Optional[List[Optional[LayerState]]] = None):
        states = list(states) if states is not None else [None] * len(self.blocks)
        out_states = []
        for blk, st in zip(self.blocks, states):
            x, ns = blk(x, st)
            out_states.append(ns)
        return x, out_states

    __call__ = forward

    def state_types(self) -> List[StateType]:
        m = {HybridLayerType.ATTENTION: StateType.KV_CACHE, HybridLayerType.DIFF_ATTENTION: StateType.NONE}
        return [m.get(b.cfg.layer_type, StateType.RECURRENT) for b in self.blocks]


class HybridModelBuilder:
    def __init__(self, config: HybridArchitectureConfig):
        self.config = config

    def build(self, seed: int = 0, device="cpu") -> HybridModel:
        return HybridModel(self.config, [HybridBlock(self.config.hidden_size, lc, seed + i, device) for i, lc in enumerate(self.config.layers)])
