"""Hugging Face checkpoints of several decoder families under ONE set of tensor names (the Llama names every loader and
quantizer of this package understands), with fused projections split on the way; plus the header-only memory estimate
and the load-and-quantize entry point that goes with it.

A family is a list of :class:`Rule` (``source`` pattern with ``{L}`` for the layer number, ``target`` template, and a
``split`` kind for fused tensors): ``qkv`` cuts ``[q | k | v]`` rows by head counts, ``gate_up`` cuts ``[gate | up]`` rows in
half, ``mlp_in`` renames a non-gated first MLP matrix to ``up_proj``.  Families: llama (= mistral), qwen2 (biases on
q / k / v), gemma (tied head), phi (Phi-3: ``qkv_proj`` / ``gate_up_proj``), phi2 (``transformer.h.N.mixer.Wqkv``), starcoder2
(``c_fc`` / ``c_proj``, LayerNorm biases); ``register_architecture`` adds more at run time.

Parity: reference ``converters/safetensors_loader.py`` (``load_config`` :132, ``estimate_memory`` :182, ``load_and_quantize`` :240,
``detect_model_type`` :594, ``map_weight_names`` :633, ``load_mapped_safetensors`` :767, ``get_supported_architectures`` :836,
``register_architecture`` :842).
"""
from __future__ import annotations

import json
import os
import re
from dataclasses import dataclass
from typing import Any, Dict, Iterable, List, Optional, Sequence, Set, Tuple, Union

import torch

from ..formats.fp4 import pick_group_size
from ..formats.safetensors_io import SafetensorsFile
from ..models.config import ModelConfig

_ATTN = "model.layers.{L}.self_attn"
_MLP = "model.layers.{L}.mlp"


@dataclass(frozen=True)
class Rule:
    source: str                    # name pattern; "{L}" stands for the layer number
    target: str                    # name template ("{L}" again); for split rules the module prefix the pieces go under
    split: str = ""                # "" | "qkv" | "gate_up" | "mlp_in"

    def regex(self) -> "re.Pattern[str]":
        return re.compile("^" + re.escape(self.source).replace(re.escape("{L}"), r"(?P<L>\d+)") + "$")


def _plain(prefix_src: str, prefix_dst: str, names: Iterable[str], kinds=("weight", "bias")) -> List[Rule]:
    return [Rule(f"{prefix_src}.{n}.{k}", f"{prefix_dst}.{n}.{k}") for n in names for k in kinds]


def _llama_rules() -> List[Rule]:
    r = [Rule("model.embed_tokens.weight", "model.embed_tokens.weight"), Rule("model.norm.weight", "model.norm.weight"),
         Rule("model.norm.bias", "model.norm.bias"), Rule("lm_head.weight", "lm_head.weight"), Rule("lm_head.bias", "lm_head.bias")]
    r += _plain(_ATTN, _ATTN, ("q_proj", "k_proj", "v_proj", "o_proj", "q_norm", "k_norm"))
    r += _plain(_MLP, _MLP, ("gate_proj", "up_proj", "down_proj"))
    r += _plain("model.layers.{L}", "model.layers.{L}", ("input_layernorm", "post_attention_layernorm", "pre_feedforward_layernorm",
                                                          "post_feedforward_layernorm"))
    return r


def _phi3_rules() -> List[Rule]:
    r = [x for x in _llama_rules() if ".q_proj." not in x.source and ".k_proj." not in x.source and ".v_proj." not in x.source
         and ".gate_proj." not in x.source and ".up_proj." not in x.source]
    r += [Rule("model.final_layernorm.weight", "model.norm.weight"), Rule("model.final_layernorm.bias", "model.norm.bias")]
    for k in ("weight", "bias"):
        r += [Rule(f"{_ATTN}.qkv_proj.{k}", f"{_ATTN}|{k}", "qkv"), Rule(f"{_MLP}.gate_up_proj.{k}", f"{_MLP}|{k}", "gate_up")]
    return r


def _phi2_rules() -> List[Rule]:
    h = "transformer.h.{L}"
    r = [Rule("transformer.embd.wte.weight", "model.embed_tokens.weight"), Rule("lm_head.linear.weight", "lm_head.weight"),
         Rule("lm_head.linear.bias", "lm_head.bias"), Rule("lm_head.ln.weight", "model.norm.weight"), Rule("lm_head.ln.bias", "model.norm.bias")]
    for k in ("weight", "bias"):
        r += [Rule(f"{h}.ln.{k}", f"model.layers.{{L}}.input_layernorm.{k}"), Rule(f"{h}.mixer.Wqkv.{k}", f"{_ATTN}|{k}", "qkv"),
              Rule(f"{h}.mixer.out_proj.{k}", f"{_ATTN}.o_proj.{k}"), Rule(f"{h}.mlp.fc1.{k}", f"{_MLP}|{k}", "mlp_in"),
              Rule(f"{h}.mlp.fc2.{k}", f"{_MLP}.down_proj.{k}")]
    return r


def _starcoder2_rules() -> List[Rule]:
    r = [x for x in _llama_rules() if ".mlp." not in x.source]
    for k in ("weight", "bias"):
        r += [Rule(f"{_MLP}.c_fc.{k}", f"{_MLP}|{k}", "mlp_in"), Rule(f"{_MLP}.c_proj.{k}", f"{_MLP}.down_proj.{k}")]
    return r


_FAMILIES: Dict[str, List[Rule]] = {
    "llama": _llama_rules(), "mistral": _llama_rules(), "qwen2": _llama_rules(), "gemma": _llama_rules(),
    "phi": _phi3_rules(), "phi2": _phi2_rules(), "starcoder2": _starcoder2_rules(),
}
_COMPILED: Dict[str, List[Tuple["re.Pattern[str]", Rule]]] = {}


def get_supported_architectures() -> List[str]:
    return list(_FAMILIES)


def register_architecture(name: str, rules: Sequence[Union[Rule, Tuple[str, str], Tuple[str, str, str]]], *, overwrite: bool = False) -> None:
    """Add (or with ``overwrite`` replace) a family.  Rules are :class:`Rule` objects or ``(source, target[, split])`` tuples
    with ``{L}`` (``{layer}`` is accepted too) for the layer number; a split rule's target is ``"<module prefix>|<weight or bias>"``."""
    if name in _FAMILIES and not overwrite:
        raise ValueError(f"architecture {name!r} is registered already (pass overwrite=True to replace it)")
    out = []
    for r in rules:
        if not isinstance(r, Rule):
            r = Rule(*[s.replace("{layer}", "{L}") if i < 2 else s for i, s in enumerate(r)])
        out.append(r)
    _FAMILIES[name] = out
    _COMPILED.pop(name, None)


def detect_model_type(state_dict_keys: Iterable[str]) -> str:
    keys = set(state_dict_keys)
    has = lambda frag: any(frag in k for k in keys)          # noqa: E731
    if any(k.startswith("transformer.h.") for k in keys):
        return "phi2"
    if has("qkv_proj") or has("gate_up_proj"):
        return "phi"
    if has("mlp.c_fc"):
        return "starcoder2"
    if has("self_attn.q_proj.bias"):
        return "qwen2"
    if "lm_head.weight" not in keys and has("model.embed_tokens"):
        return "gemma"
    return "llama"


def _cfg_get(config, key: str, default=None):
    if config is None:
        return default
    if isinstance(config, dict):
        return config.get(key, default)
    return getattr(config, key, default)


def _split_qkv(t: torch.Tensor, heads: int, kv_heads: int, head_dim: Optional[int]) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    rows = t.shape[0]
    hd = head_dim or rows // (heads + 2 * kv_heads)
    q, kv = heads * hd, kv_heads * hd
    if q + 2 * kv != rows:
        raise ValueError(f"fused qkv with {rows} rows does not match {heads} query and {kv_heads} key/value heads of size {hd}")
    return t[:q].contiguous(), t[q: q + kv].contiguous(), t[q + kv:].contiguous()


def map_weight_names(hf_state_dict: Dict[str, torch.Tensor], model_type: str = "auto", *, num_heads: Optional[int] = None,
                     num_kv_heads: Optional[int] = None, head_dim: Optional[int] = None, intermediate_size: Optional[int] = None,
                     config: Union[ModelConfig, Dict[str, Any], None] = None, strict: bool = False) -> Dict[str, torch.Tensor]:
    """Rename (and split) a state dict into the Llama names.  Head counts come from the arguments, else from ``config``; a
    fused q|k|v tensor needs them.  Names no rule covers are kept as they are (``strict`` raises instead)."""
    if model_type == "auto":
        model_type = detect_model_type(hf_state_dict.keys())
    if model_type not in _FAMILIES:
        raise ValueError(f"unknown architecture {model_type!r}; known: {get_supported_architectures()}")
    rules = _COMPILED.get(model_type)
    if rules is None:
        rules = _COMPILED[model_type] = [(r.regex(), r) for r in _FAMILIES[model_type]]
    heads = num_heads or _cfg_get(config, "num_attention_heads")
    kv_heads = num_kv_heads or _cfg_get(config, "num_key_value_heads") or heads
    head_dim = head_dim or _cfg_get(config, "head_dim")
    inter = intermediate_size or _cfg_get(config, "intermediate_size")
    out: Dict[str, torch.Tensor] = {}
    for name, t in hf_state_dict.items():
        for rx, rule in rules:
            m = rx.match(name)
            if not m:
                continue
            L = m.groupdict().get("L", "")
            target = rule.target.replace("{L}", L)
            if not rule.split:
                out[target] = t
            else:
                prefix, kind = target.split("|")
                if rule.split == "qkv":
                    if not heads:
                        raise ValueError(f"{name}: splitting a fused q|k|v tensor needs num_heads (argument or config)")
                    for part, piece in zip(("q_proj", "k_proj", "v_proj"), _split_qkv(t, int(heads), int(kv_heads), head_dim)):
                        out[f"{prefix}.{part}.{kind}"] = piece
                elif rule.split == "gate_up":
                    half = int(inter) if inter and 2 * int(inter) == t.shape[0] else t.shape[0] // 2
                    if 2 * half != t.shape[0]:
                        raise ValueError(f"{name}: {t.shape[0]} rows cannot be cut into gate and up halves")
                    out[f"{prefix}.gate_proj.{kind}"], out[f"{prefix}.up_proj.{kind}"] = t[:half].contiguous(), t[half:].contiguous()
                elif rule.split == "mlp_in":
                    out[f"{prefix}.up_proj.{kind}"] = t
                else:
                    raise ValueError(f"unknown split kind {rule.split!r}")
            break
        else:
            if strict:
                raise KeyError(f"no {model_type} rule covers {name}")
            out[name] = t
    return out


def load_config(config_path: str) -> ModelConfig:
    """``config.json`` (a path to it or to its directory) as this package's :class:`ModelConfig`."""
    path = os.path.join(config_path, "config.json") if os.path.isdir(config_path) else str(config_path)
    with open(path) as f:
        return ModelConfig.from_dict(json.load(f))


def _shards(model_path: str) -> List[str]:
    model_path = str(model_path)
    if os.path.isdir(model_path):
        files = sorted(os.path.join(model_path, f) for f in os.listdir(model_path) if f.endswith(".safetensors"))
        if not files:
            raise FileNotFoundError(f"{model_path}: no .safetensors files")
        return files
    return [model_path]


_ELEM = {"F64": 8, "F32": 4, "F16": 2, "BF16": 2, "I64": 8, "I32": 4, "U32": 4, "I16": 2, "I8": 1, "U8": 1, "BOOL": 1, "F8_E4M3": 1, "F8_E5M2": 1}


def _quantizable(name: str, shape: Sequence[int], group_size: int) -> bool:
    from ..quant.convert import should_quantize_tensor
    return len(shape) == 2 and shape[1] % 8 == 0 and shape[0] % 8 == 0 and should_quantize_tensor(name, torch.empty(tuple(int(d) for d in shape), device="meta"))


def estimate_memory(model_path: str, group_size: int = 128) -> Dict[str, float]:
    """Sizes before and after 4-bit quantization from the shard headers alone (no tensor data is read): quantizable
    matrices at half a byte per weight plus one 16-bit scale per group (the largest supported group size dividing the input width), the rest at 16 bits."""
    total = quant = 0
    qbytes = 0.0
    for path in _shards(model_path):
        f = SafetensorsFile(path)
        for k in f.keys():
            shape = f.shape(k)
            n = 1
            for d in shape:
                n *= int(d)
            total += n
            if _quantizable(k, shape, group_size):
                quant += n
                qbytes += n / 2 + 2 * n / pick_group_size(int(shape[1]), group_size)
            else:
                qbytes += 2 * n
    fp16 = 2.0 * total
    return {"fp16_gb": fp16 / 2 ** 30, "quantized_gb": qbytes / 2 ** 30, "savings_ratio": fp16 / qbytes if qbytes else 1.0,
            "total_elements": float(total), "quantized_elements": float(quant)}


def load_mapped_safetensors(path: str, model_type: str = "auto", *, config: Union[ModelConfig, Dict[str, Any], None] = None,
                            config_path: Optional[str] = None) -> Tuple[Dict[str, torch.Tensor], ModelConfig]:
    """All tensors of a file or shard directory under the Llama names, with the parsed configuration."""
    base = str(path) if os.path.isdir(str(path)) else os.path.dirname(os.path.abspath(str(path)))
    if config is None:
        config = load_config(config_path or base)
    elif isinstance(config, dict):
        config = ModelConfig.from_dict(config)
    sd: Dict[str, torch.Tensor] = {}
    for p in _shards(path):
        f = SafetensorsFile(p)
        for k in f.keys():
            sd[k] = f.get_tensor(k)
    return map_weight_names(sd, model_type, config=config), config


def load_and_quantize(model_path: str, quant_type: str = "fp4", group_size: int = 128, model_type: str = "auto",
                      device: Optional[str] = None) -> Tuple[Dict[str, Any], ModelConfig]:
    """Stream the checkpoint, map its names, and quantize every eligible matrix (``fp4``: E2M1 codes with group scales;
    ``int4``: unsigned 4-bit with scale and zero point; ``int8``; ``nf4``).  Returns ``{name: QuantizedTensor | Tensor}`` (everything
    not quantized is passed through in 16 bits) and the configuration."""
    from ..quant import rtn
    sd, cfg = load_mapped_safetensors(model_path, model_type)
    out: Dict[str, Any] = {}
    for k, t in sd.items():
        if t.is_floating_point() and _quantizable(k, t.shape, group_size):
            w = t.to(device) if device else t
            out[k] = rtn.quantize(w.float(), quant_type, pick_group_size(t.shape[1], group_size))
        else:
            out[k] = t.to(torch.float16) if t.is_floating_point() and t.dtype == torch.float32 else t
    return out, cfg
