"""EXL3-style (trellis) checkpoints: format detection, regrouping of sharded files into one directory per layer, loading
from a local directory or the Hugging Face hub, and conversion to the FP4 tile formats of this engine.

A trellis checkpoint holds, per quantized matrix, the packed code stream (``indices``), per-group ``scales`` and the sign
vectors ``su`` / ``sv`` (``formats/trellis.py``); everything else (norms, embeddings, routers) is stored as it is.  Three file
layouts occur: a single ``model.safetensors``, shards ``model-0000k-of-0000n.safetensors``, and the layer-wise layout
(``layer_NNNN/`` directories + ``base_weights.safetensors``) that loads one layer at a time.

The engine runs trellis checkpoints natively (``trellis/lm.py``); conversion to MMFP4 / marlin_fp4 is for deployments that
want one weight format: every matrix is de-quantized exactly and re-quantized to E2M1 with fp16 group scales.

Parity: reference ``metal_marlin/hf_exl3_loader.py``: ``download_exl3_model`` ``:22``, ``detect_exl3_format`` ``:54``,
``convert_sharded_to_layerwise`` ``:134``, ``load_exl3_from_hub`` ``:216``, ``list_exl3_models`` ``:269``, ``parse_model_card``
``:331``; ``metal_marlin/quantization/exl3_to_marlin.py``: ``exl3_layer_to_marlin`` ``:334``, ``convert_exl3_to_marlin`` ``:418``.
"""
from __future__ import annotations

import json
import os
import re
from typing import Dict, Iterator, List, Optional, Tuple

import torch

from ..formats import fp4 as fp4fmt
from ..formats.safetensors_io import SafetensorsFile, save_file
from ..formats.trellis import SUFFIXES, TrellisModelLoader, TrellisWeight, detect_trellis_format, tensor_key

_SHARD_RE = re.compile(r"model-(\d+)-of-(\d+)\.safetensors$")
_LAYER_RE = re.compile(r"layers[._](\d+)[._]")
_PART_RE = re.compile(r"^(.*?)(?:__|\.)(indices|scales|su|sv)$")


def detect_exl3_format(model_path: str) -> dict:
    """``{"format": "single" | "sharded" | "layerwise", "files": [...], "config": {...}, ...}`` of a checkpoint directory."""
    cfg_path = os.path.join(model_path, "config.json")
    if not os.path.exists(cfg_path):
        raise FileNotFoundError(f"config.json not found in {model_path}")
    with open(cfg_path) as f:
        config = json.load(f)
    names = sorted(os.listdir(model_path))
    layer_dirs = [os.path.join(model_path, n) for n in names if n.startswith("layer_") and os.path.isdir(os.path.join(model_path, n))]
    if layer_dirs:
        return {"format": "layerwise", "files": layer_dirs, "config": config, "num_layers": len(layer_dirs)}
    st = [n for n in names if n.endswith(".safetensors")]
    sharded = sorted((n for n in st if _SHARD_RE.search(n)), key=lambda n: int(_SHARD_RE.search(n).group(1)))
    if sharded:
        return {"format": "sharded", "files": [os.path.join(model_path, n) for n in sharded], "config": config, "num_shards": len(sharded)}
    if len(st) == 1:
        return {"format": "single", "files": [os.path.join(model_path, st[0])], "config": config}
    if not st:
        raise FileNotFoundError(f"no safetensors files in {model_path}")
    return {"format": "sharded", "files": [os.path.join(model_path, n) for n in st], "config": config, "num_shards": len(st)}


def parse_layer_index(tensor_name: str) -> Optional[int]:
    m = _LAYER_RE.search(tensor_name)
    return int(m.group(1)) if m else None


def _split_part(key: str) -> Tuple[str, Optional[str]]:
    """``"a__b__indices"`` / ``"a.b.indices"`` -> (``"a.b"``, ``"indices"``); other tensors -> (key, None)."""
    m = _PART_RE.match(key)
    if m is None:
        return key, None
    return m.group(1).replace("__", "."), m.group(2)


def convert_sharded_to_layerwise(model_path: str, out_dir: str, bits_hint: Optional[int] = None) -> dict:
    """Regroup a single-file or sharded trellis checkpoint into ``layer_NNNN/`` directories (one ``index.json`` + one
    safetensors file per matrix) plus ``base_weights.safetensors``, reading one tensor at a time."""
    info = detect_exl3_format(model_path)
    if info["format"] == "layerwise":
        return {"layers": info["num_layers"], "already_layerwise": True}
    os.makedirs(out_dir, exist_ok=True)
    where: Dict[str, str] = {}
    for fn in info["files"]:
        with SafetensorsFile(fn) as sf:
            for k in sf.keys():
                where[k] = fn
    groups: Dict[str, Dict[str, str]] = {}          # matrix name -> part -> key
    base_keys: List[str] = []
    for k in where:
        name, part = _split_part(k)
        if part is None:
            base_keys.append(k)
        else:
            groups.setdefault(name, {})[part] = k
    incomplete = [n for n, parts in groups.items() if set(parts) != set(SUFFIXES)]
    for n in incomplete:            # a tensor that merely ends in ".scales" etc. but is no trellis matrix stays a base tensor
        base_keys.extend(groups.pop(n).values())

    def get(k):
        with SafetensorsFile(where[k]) as sf:
            return sf.get_tensor(k)

    meta = {}
    qi = os.path.join(model_path, "quantization_index.json")
    if os.path.exists(qi):
        with open(qi) as f:
            meta = {e["name"]: e for e in json.load(f).get("layers", [])}
    per_layer: Dict[int, List[str]] = {}
    for name in groups:
        per_layer.setdefault(parse_layer_index(name) or 0, []).append(name)
    for li, names in sorted(per_layer.items()):
        d = os.path.join(out_dir, f"layer_{li:04d}")
        os.makedirs(d, exist_ok=True)
        entries = []
        for j, name in enumerate(sorted(names)):
            parts = {p: get(groups[name][p]) for p in SUFFIXES}
            e = meta.get(name)
            if e is None:
                out_f, in_f = parts["sv"].numel(), parts["su"].numel()
                if parts["scales"].shape[-1] == in_f and out_f != in_f:      # checkpoints that store su by output, sv by input
                    out_f, in_f = in_f, out_f
                bits = int(parts["indices"].reshape(-1)[0]) if parts["indices"].dtype == torch.uint8 else (bits_hint or 4)
                e = {"name": name, "bits": bits, "shape": [out_f, in_f], "mse": 0.0}
            save_file({tensor_key(name, p): parts[p] for p in SUFFIXES}, os.path.join(d, f"tensor_{j:04d}.safetensors"))
            entries.append({"name": name, "bits": e["bits"], "shape": list(e["shape"]), "mse": e.get("mse", 0.0)})
        with open(os.path.join(d, "index.json"), "w") as f:
            json.dump({"tensors": entries}, f)
    save_file({k: get(k) for k in base_keys}, os.path.join(out_dir, "base_weights.safetensors"))
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(info["config"], f, indent=1)
    for aux in ("tokenizer.json", "tokenizer_config.json", "generation_config.json", "special_tokens_map.json"):
        src = os.path.join(model_path, aux)
        if os.path.exists(src):
            with open(src, "rb") as a, open(os.path.join(out_dir, aux), "wb") as b:
                b.write(a.read())
    return {"layers": len(per_layer), "matrices": len(groups), "base_tensors": len(base_keys), "already_layerwise": False}


def download_exl3_model(model_id: str, local_dir: Optional[str] = None, revision: Optional[str] = None) -> str:
    """Fetch a checkpoint from the Hugging Face hub (needs ``huggingface_hub`` and network access)."""
    try:
        from huggingface_hub import snapshot_download
    except ImportError as e:          # pragma: no cover - depends on the environment
        raise RuntimeError("huggingface_hub is not installed: download the checkpoint by other means and pass its directory") from e
    return snapshot_download(model_id, local_dir=local_dir, revision=revision,
                             allow_patterns=["*.safetensors", "*.json", "tokenizer*", "*.txt"])


def load_exl3_from_hub(model_id_or_path: str, cache_dir: Optional[str] = None, layerwise: bool = True, device: Optional[str] = None):
    """Local directory or hub id -> a ready ``TrellisForCausalLM``.  Single-file and sharded checkpoints are regrouped into
    the layer-wise layout first (next to the checkpoint, ``<dir>-layerwise``) unless ``layerwise=False`` and the checkpoint
    already carries the index files the loader understands."""
    path = model_id_or_path if os.path.isdir(model_id_or_path) else download_exl3_model(model_id_or_path, cache_dir)
    info = detect_exl3_format(path)
    if info["format"] != "layerwise" and (layerwise or detect_trellis_format(path) is None):
        out = path.rstrip("/") + "-layerwise"
        if not os.path.isdir(os.path.join(out, "layer_0000")):
            convert_sharded_to_layerwise(path, out)
        path = out
    from ..trellis.lm import TrellisForCausalLM
    return TrellisForCausalLM.from_pretrained(path, device=device)


def list_exl3_models(author: Optional[str] = None, search: str = "exl3", limit: int = 50) -> List[dict]:
    """Hub search for trellis-quantized repositories (needs ``huggingface_hub`` and network access)."""
    try:
        from huggingface_hub import HfApi
    except ImportError as e:          # pragma: no cover
        raise RuntimeError("huggingface_hub is not installed") from e
    return [{"id": m.id, "downloads": getattr(m, "downloads", None), "likes": getattr(m, "likes", None), **parse_model_card(m.id)}
            for m in HfApi().list_models(author=author, search=search, limit=limit)]


def parse_model_card(model_id: str) -> dict:
    """What a repository name tells: base model and bits per weight (``org/Llama-3-8B-exl3-4.0bpw`` -> 4.0)."""
    name = model_id.split("/")[-1]
    m = re.search(r"(\d+(?:\.\d+)?)\s*bpw", name, re.I)
    base = re.sub(r"[-_.]?(exl3|\d+(?:\.\d+)?bpw|h\d+)", "", name, flags=re.I).strip("-_.")
    return {"base_model": base, "bpw": float(m.group(1)) if m else None, "is_exl3": "exl3" in name.lower()}


# ---------------------------------------------------------------------------------------------------- to FP4
def exl3_layer_to_marlin(tw: TrellisWeight, group_size: int = 128, layout: str = "marlin_fp4") -> Tuple[torch.Tensor, torch.Tensor, float]:
    """One trellis matrix -> packed FP4 words + fp16 group scales in the ``marlin_fp4`` (``[in / 8, out]``) or ``mmfp4``
    (``[out, in / 8]``) checkpoint layout, and the relative RMS error of the re-quantization."""
    w = tw.dequantize(torch.float32)
    gs = fp4fmt.pick_group_size(w.shape[1], group_size)
    codes, scales = fp4fmt.quantize_codes(w, gs)
    err = float((fp4fmt.dequantize_codes(codes, scales) - w).pow(2).mean().sqrt() / w.pow(2).mean().sqrt().clamp_min(1e-12))
    packed, sc = fp4fmt.pack_marlin_fp4(codes, scales) if layout == "marlin_fp4" else fp4fmt.pack_mmfp4(codes, scales)
    return packed, sc, err


def iter_exl3_float_tensors(path: str) -> Iterator[Tuple[str, torch.Tensor]]:
    """``(name, tensor)`` of a trellis checkpoint with every quantized matrix de-quantized (bf16) and every other tensor as
    stored - the stream a float-checkpoint converter expects."""
    ld = TrellisModelLoader(path)
    seen = set()
    for name in ld.weight_names():
        yield name, ld.load_weight(name).dequantize(torch.float32).to(torch.bfloat16)
        for p in SUFFIXES:
            seen.add(tensor_key(name, p))
            seen.add(tensor_key(name, p, dotted=True))
    for k in list(ld._where):
        if k not in seen:
            yield k, ld.load_tensor(k)


def convert_exl3_to_marlin(exl3_path: str, output_path: str, fmt: str = "mmfp4", group_size: int = 128, verbose: bool = False) -> dict:
    """Whole checkpoint: trellis (any of the three file layouts) -> MMFP4 shards or one ``marlin_fp4`` file, config and
    tokenizer files copied along.  Returns ``{"layers_converted", "total_params", "original_bytes", "converted_bytes",
    "compression_ratio", "mean_rel_rmse", "errors"}``."""
    from ..quant.convert import convert_model
    stats = {"layers_converted": 0, "total_params": 0, "original_bytes": 0, "converted_bytes": 0, "compression_ratio": 1.0,
             "mean_rel_rmse": 0.0, "errors": []}
    if not os.path.isdir(exl3_path):
        stats["errors"].append(f"input path does not exist: {exl3_path}")
        return stats
    src = exl3_path
    if detect_trellis_format(src) is None:                  # single file / plain shards: regroup first
        src = os.path.join(output_path, "_layerwise")
        convert_sharded_to_layerwise(exl3_path, src)
    ld = TrellisModelLoader(src)
    for name in ld.weight_names():
        e = ld.meta[name]
        n = int(e["shape"][0]) * int(e["shape"][1])
        stats["total_params"] += n
        stats["original_bytes"] += n * int(e["bits"]) // 8
    rep = convert_model(src, output_path, fmt, group_size, verbose=verbose, tensors=iter_exl3_float_tensors(src))
    cfg_src = os.path.join(exl3_path, "config.json")
    if os.path.exists(cfg_src) and not os.path.exists(os.path.join(output_path, "config.json")):
        with open(cfg_src) as f:
            cfg = json.load(f)
        with open(os.path.join(output_path, "config.json"), "w") as f:
            json.dump(cfg, f, indent=1)
    stats["layers_converted"] = rep["quantized"]
    stats["mean_rel_rmse"] = rep["mean_rel_rmse"]
    stats["converted_bytes"] = stats["total_params"] // 2 + 2 * (stats["total_params"] // max(1, group_size))
    stats["compression_ratio"] = stats["original_bytes"] / max(1, stats["converted_bytes"])
    return stats
