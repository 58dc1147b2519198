"""NeMo / Megatron-LM GPT checkpoints to Hugging Face (Llama-style) tensor names and layouts.

A ``.nemo`` archive is a tar file with ``model_config.yaml`` and ``model_weights.ckpt`` (a PyTorch state dict, possibly
under ``model_weights/``); the Megatron layout fuses q/k/v into ``linear_qkv`` (interleaved per KV group:
``[q_0 .. q_{g-1}, k, v]`` for every group) and gate / up into ``linear_fc1`` (gate rows first).  ``convert_state_dict``
undoes both and renames to ``model.layers.N.self_attn.{q,k,v,o}_proj`` / ``mlp.{gate,up,down}_proj`` so every loader and
quantizer of this package applies.

Parity: reference ``metal_marlin/converters`` NeMo -> PyTorch path.
"""
from __future__ import annotations

import io
import re
import tarfile
from typing import Dict, Optional, Tuple

import torch
import yaml


def split_fused_qkv(w: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Megatron ``linear_qkv`` ``[(Hq + 2 Hkv) * D, hidden]`` (grouped per KV head) -> q ``[Hq * D, hidden]``, k, v."""
    g = num_heads // num_kv_heads
    rest = w.shape[1:]
    x = w.reshape(num_kv_heads, g + 2, head_dim, *rest)
    q = x[:, :g].reshape(num_heads * head_dim, *rest)
    k = x[:, g].reshape(num_kv_heads * head_dim, *rest)
    v = x[:, g + 1].reshape(num_kv_heads * head_dim, *rest)
    return q.contiguous(), k.contiguous(), v.contiguous()


_RULES = [
    (r"^(?:model\.)?embedding\.word_embeddings\.weight$", "model.embed_tokens.weight"),
    (r"^(?:model\.)?decoder\.final_layernorm\.weight$", "model.norm.weight"),
    (r"^(?:model\.)?output_layer\.weight$", "lm_head.weight"),
    (r"^(?:model\.)?decoder\.layers\.(\d+)\.self_attention\.linear_proj\.weight$", r"model.layers.\1.self_attn.o_proj.weight"),
    (r"^(?:model\.)?decoder\.layers\.(\d+)\.self_attention\.linear_qkv\.layer_norm_weight$", r"model.layers.\1.input_layernorm.weight"),
    (r"^(?:model\.)?decoder\.layers\.(\d+)\.input_layernorm\.weight$", r"model.layers.\1.input_layernorm.weight"),
    (r"^(?:model\.)?decoder\.layers\.(\d+)\.mlp\.linear_fc1\.layer_norm_weight$", r"model.layers.\1.post_attention_layernorm.weight"),
    (r"^(?:model\.)?decoder\.layers\.(\d+)\.pre_mlp_layernorm\.weight$", r"model.layers.\1.post_attention_layernorm.weight"),
    (r"^(?:model\.)?decoder\.layers\.(\d+)\.mlp\.linear_fc2\.weight$", r"model.layers.\1.mlp.down_proj.weight"),
    (r"^(?:model\.)?decoder\.layers\.(\d+)\.self_attention\.q_layernorm\.weight$", r"model.layers.\1.self_attn.q_norm.weight"),
    (r"^(?:model\.)?decoder\.layers\.(\d+)\.self_attention\.k_layernorm\.weight$", r"model.layers.\1.self_attn.k_norm.weight"),
]
_QKV = re.compile(r"^(?:model\.)?decoder\.layers\.(\d+)\.self_attention\.linear_qkv\.(weight|bias)$")
_FC1 = re.compile(r"^(?:model\.)?decoder\.layers\.(\d+)\.mlp\.linear_fc1\.weight$")


def convert_state_dict(sd: Dict[str, torch.Tensor], num_heads: int, num_kv_heads: Optional[int] = None, head_dim: Optional[int] = None,
                       gated_mlp: bool = True) -> Dict[str, torch.Tensor]:
    """Megatron-core GPT names -> HF Llama names; fused tensors are split.  Unknown keys (``_extra_state`` blobs, rotary
    caches) are dropped."""
    num_kv_heads = num_kv_heads or num_heads
    out: Dict[str, torch.Tensor] = {}
    for k, v in sd.items():
        if not isinstance(v, torch.Tensor) or k.endswith("_extra_state"):
            continue
        m = _QKV.match(k)
        if m:
            hd = head_dim or v.shape[0] // (num_heads + 2 * num_kv_heads)
            q, kk, vv = split_fused_qkv(v, num_heads, num_kv_heads, hd)
            for name, t in (("q_proj", q), ("k_proj", kk), ("v_proj", vv)):
                out[f"model.layers.{m.group(1)}.self_attn.{name}.{m.group(2)}"] = t
            continue
        m = _FC1.match(k)
        if m:
            if gated_mlp:
                gate, up = v.chunk(2, 0)
                out[f"model.layers.{m.group(1)}.mlp.gate_proj.weight"] = gate.contiguous()
                out[f"model.layers.{m.group(1)}.mlp.up_proj.weight"] = up.contiguous()
            else:
                out[f"model.layers.{m.group(1)}.mlp.up_proj.weight"] = v
            continue
        for pat, rep in _RULES:
            if re.match(pat, k):
                out[re.sub(pat, rep, k)] = v
                break
    return out


def hf_config_from_nemo(cfg: Dict) -> Dict:
    """The fields of ``model_config.yaml`` a Llama-style ``config.json`` needs."""
    heads = int(cfg.get("num_attention_heads", 32))
    hidden = int(cfg.get("hidden_size", 4096))
    return {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_size": hidden, "num_attention_heads": heads,
            "num_key_value_heads": int(cfg.get("num_query_groups", heads) or heads), "num_hidden_layers": int(cfg.get("num_layers", 32)),
            "intermediate_size": int(cfg.get("ffn_hidden_size", 4 * hidden)), "head_dim": int(cfg.get("kv_channels") or hidden // heads),
            "rms_norm_eps": float(cfg.get("layernorm_epsilon", 1e-5)), "rope_theta": float(cfg.get("rotary_base", 10000.0)),
            "max_position_embeddings": int(cfg.get("max_position_embeddings", cfg.get("encoder_seq_length", 4096))),
            "vocab_size": int(cfg.get("padded_vocab_size", cfg.get("vocab_size", 32000))), "tie_word_embeddings": bool(cfg.get("share_embeddings_and_output_weights", False))}


def load_nemo(path: str) -> Tuple[Dict[str, torch.Tensor], Dict]:
    """(HF-named state dict, HF-style config) from a ``.nemo`` archive."""
    cfg, sd = {}, None
    with tarfile.open(path) as tf:
        for m in tf.getmembers():
            base = m.name.split("/")[-1]
            if base == "model_config.yaml":
                cfg = yaml.safe_load(tf.extractfile(m).read()) or {}
            elif base in ("model_weights.ckpt", "model_weights.pt"):
                sd = torch.load(io.BytesIO(tf.extractfile(m).read()), map_location="cpu", weights_only=True)
    if sd is None:
        raise ValueError(f"{path}: no model_weights.ckpt inside the archive")
    sd = sd.get("state_dict", sd)
    hf = hf_config_from_nemo(cfg)
    return convert_state_dict(sd, hf["num_attention_heads"], hf["num_key_value_heads"], hf["head_dim"],
                              gated_mlp=str(cfg.get("activation", "fast-swiglu")).endswith("glu")), hf


def convert_nemo_to_pytorch(nemo_path: str, output_path: str, *, extract_config_only: bool = False, config_output: Optional[str] = None,
                            use_safetensors: bool = True) -> Dict:
    """A ``.nemo`` archive to a standard checkpoint: Hugging Face tensor names in ``output_path`` (``.safetensors``, or a
    ``torch.save`` file when ``use_safetensors`` is off or the name ends in ``.pt`` / ``.bin``; a directory gets ``model.safetensors`` and
    ``config.json``).  ``config_output`` also writes the derived configuration as JSON; ``extract_config_only`` stops after that.
    Returns ``{"config", "num_tensors", "num_parameters", "output"}`` (reference ``converters/nemo_to_pytorch.py:173``)."""
    import json
    import os
    nemo_path, output_path = str(nemo_path), str(output_path)
    if not os.path.isfile(nemo_path):
        raise FileNotFoundError(f"NeMo file not found: {nemo_path}")
    if not nemo_path.endswith(".nemo"):
        raise ValueError(f"expected a .nemo archive, got {nemo_path}")
    if extract_config_only:
        with tarfile.open(nemo_path) as tf:
            raw = next((yaml.safe_load(tf.extractfile(m).read()) or {} for m in tf.getmembers() if m.name.split("/")[-1] == "model_config.yaml"), None)
        if raw is None:
            raise FileNotFoundError(f"{nemo_path}: no model_config.yaml inside the archive")
        sd, hf = {}, hf_config_from_nemo(raw)
    else:
        sd, hf = load_nemo(nemo_path)
    if config_output:
        os.makedirs(os.path.dirname(os.path.abspath(config_output)), exist_ok=True)
        with open(config_output, "w") as f:
            json.dump(hf, f, indent=1)
    info = {"config": hf, "num_tensors": len(sd), "num_parameters": int(sum(t.numel() for t in sd.values())), "output": None}
    if extract_config_only:
        return info
    as_dir = os.path.isdir(output_path) or not os.path.splitext(output_path)[1]
    if as_dir:
        os.makedirs(output_path, exist_ok=True)
        with open(os.path.join(output_path, "config.json"), "w") as f:
            json.dump(hf, f, indent=1)
        target = os.path.join(output_path, "model.safetensors" if use_safetensors else "pytorch_model.bin")
    else:
        os.makedirs(os.path.dirname(os.path.abspath(output_path)), exist_ok=True)
        target = output_path
    if use_safetensors and target.endswith(".safetensors"):
        from ..formats.safetensors_io import save_file
        save_file({k: v.contiguous() for k, v in sd.items()}, target, metadata={"format": "pt"})
    else:
        torch.save(sd, target)
    info["output"] = target
    return info
