"""Shape contract of the dense Qwen3.6-27B hybrid (Gated DeltaNet layers with a full-attention layer every fourth) and the
decode-path assumptions this framework makes for it on B200.

The profile is data: dimensions parsed from a Hugging Face ``config.json`` (the text part of a multimodal config), the layer
pattern, detection of the supported model (the 35B-A3B MoE sibling is not it), and a payload for validation scripts.  The
hardware part states how the decode path is laid out on this GPU rather than on the reference's.

Parity: reference ``qwen36_27b_profile.py`` (``Qwen36DeltaNetProfile`` :53, ``Qwen36FullAttentionProfile`` :82, ``Qwen36DenseMLPProfile`` :103,
``Qwen36ModelProfile`` :108, ``profile_from_hf_config`` :158, ``load_profile_from_config_file`` :193, ``shape_contract_payload`` :201,
``is_qwen36_27b_profile`` :221, ``is_qwen36_27b_config`` :235, ``validate_supported_profile`` :250; its ``AppleSiliconDecodeProfile`` :23
is ``B200DecodeProfile`` here).
"""
from __future__ import annotations

import json
from dataclasses import asdict, dataclass, field
from typing import Any, Dict, List, Tuple

MODEL_ID = "Qwen/Qwen3.6-27B"


@dataclass(frozen=True)
class B200DecodeProfile:
    warp_size: int = 32
    preferred_group_size: int = 128
    int4_pack_factor: int = 8                  # codes per 32-bit word
    sms: int = 148
    fp32_accumulation: bool = True
    keep_weights_compressed: bool = True
    decode_in_cuda_graph: bool = True
    target_launches_per_layer: int = 9
    rules: Tuple[str, ...] = (
        "Decode is weight-streaming: INT4 / FP4 words stay packed in HBM and are expanded in registers by the GEMV kernels; nothing is "
        "materialised in 16 bits.",
        "Dot products, soft-max statistics and the recurrent state update accumulate in fp32; the state of the gated delta rule is "
        "kept in fp32 in its pool.",
        "Projections that read the same activation run as one launch over a concatenated weight; residual add, RMSNorm and SwiGLU "
        "ride in the GEMV prologue / epilogue.",
        "The whole step is captured in a CUDA graph per batch bucket; the recurrent step kernel and the paged attention kernel "
        "are both graph-safe (no host reads).",
        "Prompt passes of more than a few dozen tokens go to the tcgen05 GEMM and the scan kernel (one CTA per batch row and "
        "value head) instead.",
        "Benchmarks on template weights are launch evidence only; quality claims need per-layer artifacts and perplexity parity.",
    )


@dataclass(frozen=True)
class Qwen36DeltaNetProfile:
    key_heads: int = 16
    value_heads: int = 48
    key_dim: int = 128
    value_dim: int = 128
    conv_kernel_dim: int = 4

    @property
    def q_features(self) -> int:
        return self.key_heads * self.key_dim

    @property
    def k_features(self) -> int:
        return self.key_heads * self.key_dim

    @property
    def v_features(self) -> int:
        return self.value_heads * self.value_dim

    @property
    def beta_features(self) -> int:
        return self.value_heads

    @property
    def state_elements(self) -> int:
        return self.value_heads * self.key_dim * self.value_dim


@dataclass(frozen=True)
class Qwen36FullAttentionProfile:
    heads: int = 24
    kv_heads: int = 4
    head_dim: int = 256
    rotary_dim: int = 64

    @property
    def q_features(self) -> int:
        return self.heads * self.head_dim * 2              # the query projection also emits the output gate

    @property
    def kv_features(self) -> int:
        return self.kv_heads * self.head_dim

    @property
    def o_features(self) -> int:
        return self.heads * self.head_dim


@dataclass(frozen=True)
class Qwen36DenseMLPProfile:
    intermediate_size: int = 17408


@dataclass(frozen=True)
class Qwen36ModelProfile:
    model_id: str = MODEL_ID
    model_type: str = "qwen3_5"
    text_model_type: str = "qwen3_5_text"
    hidden_size: int = 5120
    num_hidden_layers: int = 64
    vocab_size: int = 248320
    max_position_embeddings: int = 262144
    full_attention_interval: int = 4
    group_size: int = 128
    rms_norm_eps: float = 1e-6
    delta: Qwen36DeltaNetProfile = field(default_factory=Qwen36DeltaNetProfile)
    attention: Qwen36FullAttentionProfile = field(default_factory=Qwen36FullAttentionProfile)
    dense_mlp: Qwen36DenseMLPProfile = field(default_factory=Qwen36DenseMLPProfile)
    hardware: B200DecodeProfile = field(default_factory=B200DecodeProfile)

    @property
    def full_attention_layer_indices(self) -> List[int]:
        k = self.full_attention_interval
        return [i for i in range(self.num_hidden_layers) if i % k == k - 1]

    @property
    def num_full_attention_layers(self) -> int:
        return len(self.full_attention_layer_indices)

    @property
    def num_linear_attention_layers(self) -> int:
        return self.num_hidden_layers - self.num_full_attention_layers

    @property
    def layer_types(self) -> List[str]:
        full = set(self.full_attention_layer_indices)
        return ["full_attention" if i in full else "linear_attention" for i in range(self.num_hidden_layers)]

    def recurrent_state_bytes(self, batch: int = 1, dtype_bytes: int = 4) -> int:
        """State of all linear-attention layers for ``batch`` sequences (fp32 by default), convolution tails included."""
        d = self.delta
        conv = (d.q_features + d.k_features + d.v_features) * (d.conv_kernel_dim - 1) * 2
        return batch * self.num_linear_attention_layers * (d.state_elements * dtype_bytes + conv)

    def kv_bytes_per_token(self, dtype_bytes: int = 2) -> int:
        return 2 * self.num_full_attention_layers * self.attention.kv_features * dtype_bytes

    def weight_elements(self) -> int:
        h, d, a = self.hidden_size, self.delta, self.attention
        lin = h * (d.q_features + d.k_features + 2 * d.v_features + 2 * d.beta_features) + d.v_features * h
        full = h * (a.q_features + 2 * a.kv_features) + a.o_features * h
        mlp = 3 * h * self.dense_mlp.intermediate_size
        return (self.num_linear_attention_layers * (lin + mlp) + self.num_full_attention_layers * (full + mlp) + 2 * h * self.vocab_size)

    def to_model_config(self):
        """The engine configuration with these dimensions (the query's output gate and the partial rotary width are not
        modelled by the shared decoder: it runs the layer pattern with a plain query projection and full-width rotation)."""
        from .config import ModelConfig
        return ModelConfig(model_type="qwen3_next", vocab_size=self.vocab_size, hidden_size=self.hidden_size, num_hidden_layers=self.num_hidden_layers,
                           num_attention_heads=self.attention.heads, num_key_value_heads=self.attention.kv_heads, head_dim=self.attention.head_dim,
                           intermediate_size=self.dense_mlp.intermediate_size, rms_norm_eps=self.rms_norm_eps, rope_theta=1e7,
                           max_position_embeddings=self.max_position_embeddings, qk_norm=True, layer_types=self.layer_types,
                           linear_num_key_heads=self.delta.key_heads, linear_num_value_heads=self.delta.value_heads,
                           linear_key_head_dim=self.delta.key_dim, linear_value_head_dim=self.delta.value_dim, group_size=self.group_size)


QWEN36_27B_PROFILE = Qwen36ModelProfile()


def _text(config: Dict[str, Any]) -> Dict[str, Any]:
    t = config.get("text_config")
    return t if isinstance(t, dict) else config


def profile_from_hf_config(config: Dict[str, Any]) -> Qwen36ModelProfile:
    t = _text(config)
    head_dim = int(t["head_dim"])
    interval = t.get("full_attention_interval")
    if interval is None:                                     # derive it from an explicit layer list
        types = list(t["layer_types"])
        full = [i for i, k in enumerate(types) if k == "full_attention"]
        interval = full[0] + 1 if full else len(types) + 1
    return Qwen36ModelProfile(
        model_id=str(config.get("_name_or_path") or MODEL_ID), model_type=str(config.get("model_type", t.get("model_type", "qwen3_5"))),
        text_model_type=str(t.get("model_type", "qwen3_5_text")), hidden_size=int(t["hidden_size"]), num_hidden_layers=int(t["num_hidden_layers"]),
        vocab_size=int(t["vocab_size"]), max_position_embeddings=int(t["max_position_embeddings"]), full_attention_interval=int(interval),
        rms_norm_eps=float(t.get("rms_norm_eps", 1e-6)),
        delta=Qwen36DeltaNetProfile(int(t["linear_num_key_heads"]), int(t["linear_num_value_heads"]), int(t["linear_key_head_dim"]),
                                    int(t["linear_value_head_dim"]), int(t.get("linear_conv_kernel_dim", 4))),
        attention=Qwen36FullAttentionProfile(int(t["num_attention_heads"]), int(t["num_key_value_heads"]), head_dim,
                                             int(float(t.get("partial_rotary_factor", 0.25)) * head_dim)),
        dense_mlp=Qwen36DenseMLPProfile(int(t["intermediate_size"])))


def load_profile_from_config_file(path: str) -> Qwen36ModelProfile:
    with open(path, encoding="utf-8") as f:
        data = json.load(f)
    if not isinstance(data, dict):
        raise ValueError(f"expected a JSON object in {path}")
    return profile_from_hf_config(data)


def shape_contract_payload(profile: Qwen36ModelProfile = QWEN36_27B_PROFILE) -> Dict[str, Any]:
    p = asdict(profile)
    p.update({"model_label": "Qwen 3.6 27B", "mlp_kind": "dense", "weights_loaded": False, "layer_types": profile.layer_types,
              "num_full_attention_layers": profile.num_full_attention_layers, "num_linear_attention_layers": profile.num_linear_attention_layers,
              "full_attention_layer_indices": profile.full_attention_layer_indices, "weight_elements": profile.weight_elements(),
              "kv_bytes_per_token": profile.kv_bytes_per_token(), "recurrent_state_bytes_per_sequence": profile.recurrent_state_bytes(1)})
    return p


def is_qwen36_27b_profile(profile: Qwen36ModelProfile) -> bool:
    e = QWEN36_27B_PROFILE
    return (profile.hidden_size, profile.num_hidden_layers, profile.vocab_size, profile.full_attention_interval, profile.dense_mlp, profile.delta,
            profile.attention) == (e.hidden_size, e.num_hidden_layers, e.vocab_size, e.full_attention_interval, e.dense_mlp, e.delta, e.attention)


def is_qwen36_27b_config(config: Dict[str, Any], model_name: str = "") -> bool:
    """The dense 27B model only: a name that says 35B / A3B is refused even if some dimensions agree."""
    try:
        profile = profile_from_hf_config(config)
    except (KeyError, TypeError, ValueError):
        return False
    names = f"{model_name} {config.get('_name_or_path', '')}".lower()
    if "qwen3.6-35b" in names or "a3b" in names or _text(config).get("num_experts"):
        return False
    return is_qwen36_27b_profile(profile)


def validate_supported_profile(profile: Qwen36ModelProfile) -> None:
    if is_qwen36_27b_profile(profile):
        return
    e = QWEN36_27B_PROFILE
    diffs = [f"{k}: {getattr(profile, k)} (expected {getattr(e, k)})" for k in ("hidden_size", "num_hidden_layers", "vocab_size", "full_attention_interval",
                                                                               "dense_mlp", "delta", "attention") if getattr(profile, k) != getattr(e, k)]
    raise ValueError("not the Qwen3.6-27B shape contract: " + "; ".join(diffs))
