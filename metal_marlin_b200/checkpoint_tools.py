"""Checkpoint maintenance: verify and repair MMFP4 / marlin-FP4 checkpoints, migrate trellis containers between the
layer-directory (v2) and sharded (v3) layouts, extract the unquantized (base) and router tensors, 2:4-prune float
checkpoints, and cut a shallow draft model out of a checkpoint for speculative decoding.

Parity: reference ``scripts/repair_mmfp4_checkpoint.py`` / ``fix_mmfp4_base_weights.py`` (index vs shard contents, weight /
scale pairing, missing base tensors), ``scripts/migrate_trellis_v2_to_v3.py``, ``scripts/extract_base_weights.py`` /
``extract_router_weights.py``, ``scripts/prune_model.py`` (2:4 magnitude pruning), ``scripts/create_draft_weights.py`` (draft
for speculative decoding).  Everything here is file work on the host; the CLI exposes it as ``metal-marlin checkpoint ...``.
"""
from __future__ import annotations

import json
import os
import re
import shutil
from typing import Dict, Iterable, List, Optional, Tuple

import torch

from .formats.mmfp4_loader import SCALE_SUFFIXES, WEIGHT_SUFFIXES, MMFP4ModelLoader, extract_layer_index
from .formats.safetensors_io import SafetensorsFile, save_file
from .formats.trellis import SUFFIXES as TRELLIS_PARTS
from .formats.trellis import TrellisModelLoader, save_trellis_v2, save_trellis_v3, tensor_key

_SIDE_FILES = ("config.json", "generation_config.json", "tokenizer.json", "tokenizer_config.json", "tokenizer.model",
               "special_tokens_map.json", "vocab.json", "merges.txt", "quantization_config.json", "chat_template.jinja")


def _copy_side_files(src: str, dst: str, skip: Iterable[str] = ()) -> List[str]:
    done = []
    for f in _SIDE_FILES:
        if f not in skip and os.path.isfile(os.path.join(src, f)):
            shutil.copy2(os.path.join(src, f), os.path.join(dst, f))
            done.append(f)
    return done


def _shards(path: str) -> List[str]:
    return sorted(f for f in os.listdir(path) if f.endswith(".safetensors"))


# ------------------------------------------------------------------------------------------------ MMFP4 verify / repair
def verify_mmfp4_checkpoint(path: str, check_values: bool = True) -> Dict:
    """Structural check of an MMFP4 / marlin-FP4 checkpoint directory.  Reports: keys the index names but no shard holds
    (``missing``), tensors no index entry names (``orphans``), index entries pointing at the wrong shard (``misplaced``),
    packed weights without scales and scales without weights (``unpaired``), weight / scale shapes that do not fit each
    other (``shape_mismatch``), non-finite scales (``bad_scales``), and layers without norm tensors (``missing_base``)."""
    idx_path = os.path.join(path, "model.safetensors.index.json")
    index = {}
    if os.path.exists(idx_path):
        with open(idx_path) as f:
            index = dict(json.load(f).get("weight_map", {}))
    actual: Dict[str, str] = {}
    shapes: Dict[str, Tuple[Tuple[int, ...], str]] = {}
    for s in _shards(path):
        with SafetensorsFile(os.path.join(path, s)) as sf:
            for k in sf.keys():
                actual[k] = s
                shapes[k] = (tuple(sf.shape(k)), sf.dtype_str(k))
    rep = {"path": path, "shards": len(_shards(path)), "tensors": len(actual), "indexed": len(index), "missing": [], "orphans": [],
           "misplaced": [], "unpaired": [], "shape_mismatch": [], "bad_scales": [], "missing_base": []}
    if index:
        rep["missing"] = sorted(k for k in index if k not in actual)
        rep["orphans"] = sorted(k for k in actual if k not in index)
        rep["misplaced"] = sorted(k for k in index if k in actual and actual[k] != index[k])

    def base_of(key: str, suffixes) -> Optional[str]:
        for suf in sorted(suffixes, key=len, reverse=True):
            if key.endswith(suf):
                return key[: -len(suf)]
        return None
    packed = {base_of(k, WEIGHT_SUFFIXES): k for k, (_s, dt) in shapes.items() if dt in ("U32", "I32") and base_of(k, WEIGHT_SUFFIXES)}
    scales = {base_of(k, SCALE_SUFFIXES): k for k in shapes if base_of(k, SCALE_SUFFIXES)}
    for b, k in packed.items():
        if b not in scales:
            rep["unpaired"].append(k)
    for b, k in scales.items():
        if b not in packed:
            rep["unpaired"].append(k)
    for b in sorted(set(packed) & set(scales)):
        ws, ss = shapes[packed[b]][0], shapes[scales[b]][0]
        ok = len(ws) == len(ss) and len(ws) in (2, 3)
        if ok:
            (o1, i8), (a, c) = ws[-2:], ss[-2:]
            row_packed = a == o1 and c > 0 and (i8 * 8) % c == 0                       # [out, in / 8] with scales [out, groups]
            row_packed_t = c == o1 and a > 0 and (i8 * 8) % a == 0                     # ... or scales [groups, out]
            col_packed = c == i8 and a > 0 and (o1 * 8) % a == 0                       # [in / 8, out] with scales [groups, out]
            ok = row_packed or row_packed_t or col_packed
        if not ok:
            rep["shape_mismatch"].append({"weight": packed[b], "weight_shape": list(ws), "scales": scales[b], "scales_shape": list(ss)})
        if check_values:
            with SafetensorsFile(os.path.join(path, actual[scales[b]])) as sf:
                if not bool(torch.isfinite(sf.get_tensor(scales[b]).float()).all()):
                    rep["bad_scales"].append(scales[b])
    layers = sorted({li for li in (extract_layer_index(k) for k in actual) if li is not None})
    for li in layers:
        if not any(extract_layer_index(k) == li and "norm" in k for k in actual):
            rep["missing_base"].append(f"layer {li}: no norm tensor")
    if layers and not any("embed_tokens" in k for k in actual):
        rep["missing_base"].append("embed_tokens")
    rep["ok"] = not any(rep[k] for k in ("missing", "misplaced", "unpaired", "shape_mismatch", "bad_scales", "missing_base"))
    return rep


def repair_mmfp4_checkpoint(path: str, base_from: Optional[str] = None, dry_run: bool = False) -> Dict:
    """Fix what can be fixed in place: rebuild ``model.safetensors.index.json`` from the shard contents (covers missing,
    orphaned and misplaced entries), replace non-finite scales by zero (the affected groups de-quantize to zero instead of
    poisoning a layer), and - given ``base_from``, a float checkpoint of the same model - add the base tensors (norms,
    embeddings, router gates, biases) that are absent, in an extra shard.  Returns the report before and after."""
    before = verify_mmfp4_checkpoint(path)
    actions = []
    if dry_run:
        return {"before": before, "actions": ["dry run"], "after": before}
    for key in before["bad_scales"]:
        shard = None
        for s in _shards(path):
            with SafetensorsFile(os.path.join(path, s)) as sf:
                if key in sf.keys():
                    shard = s
                    tensors = {k: sf.get_tensor(k).clone() for k in sf.keys()}
                    break
        if shard is not None:
            t = tensors[key]
            tensors[key] = torch.where(torch.isfinite(t.float()), t, torch.zeros_like(t))
            save_file(tensors, os.path.join(path, shard))
            actions.append(f"zeroed non-finite scales in {key}")
    if base_from is not None:
        have = set()
        for s in _shards(path):
            with SafetensorsFile(os.path.join(path, s)) as sf:
                have.update(sf.keys())
        add = {}
        src = MMFP4ModelLoader(base_from, prefetch_workers=0)
        for k in src.tensor_names():
            if k in have or _is_linear_weight(k, src):
                continue
            add[k] = src.load_tensor(k)
        src.close()
        if add:
            save_file(add, os.path.join(path, "model-base-weights.safetensors"))
            actions.append(f"added {len(add)} base tensors from {base_from}")
    weight_map = {}
    for s in _shards(path):
        with SafetensorsFile(os.path.join(path, s)) as sf:
            for k in sf.keys():
                weight_map[k] = s
    idx_path = os.path.join(path, "model.safetensors.index.json")
    if len(_shards(path)) > 1 or os.path.exists(idx_path):
        meta = {}
        if os.path.exists(idx_path):
            with open(idx_path) as f:
                meta = json.load(f).get("metadata", {})
        with open(idx_path, "w") as f:
            json.dump({"metadata": meta, "weight_map": weight_map}, f, indent=1, sort_keys=True)
        actions.append(f"rewrote the index ({len(weight_map)} tensors)")
    return {"before": before, "actions": actions, "after": verify_mmfp4_checkpoint(path)}


def _is_linear_weight(key: str, loader) -> bool:
    """2-D projection weights (what quantization replaces): not embeddings, norms, router gates, biases."""
    if not key.endswith(".weight"):
        return False
    if any(s in key for s in ("norm", "embed_tokens", "mlp.gate.weight", "router", "e_score_correction")):
        return False
    fname = loader.weight_map[key]
    return len(loader._file(fname).shape(key)) == 2 and "lm_head" not in key


# ------------------------------------------------------------------------------------------------ extraction
ROUTER_PATTERN = re.compile(r"(mlp\.gate\.weight|mlp\.gate\.e_score_correction_bias|\.router\.|block_sparse_moe\.gate\.weight)")


def extract_base_weights(path: str, out_file: str, routers: bool = False) -> Dict:
    """Write the unquantized tensors of a checkpoint (float or quantized) into one safetensors file: everything that is not
    a packed weight, its scales / metadata, or a float projection matrix.  ``routers=True`` keeps only the MoE router tensors
    (gate weights, correction biases)."""
    ld = MMFP4ModelLoader(path, prefetch_workers=0)
    out = {}
    for k in ld.tensor_names():
        dt = ld._file(ld.weight_map[k]).dtype_str(k)
        if dt in ("U32", "I32") or k.endswith(SCALE_SUFFIXES) or k.endswith((".group_size", ".hadamard_block_size")):
            continue
        if _is_linear_weight(k, ld):
            continue
        if routers != bool(ROUTER_PATTERN.search(k)) and routers:
            continue
        out[k] = ld.load_tensor(k)
    ld.close()
    os.makedirs(os.path.dirname(os.path.abspath(out_file)), exist_ok=True)
    save_file(out, out_file)
    return {"file": out_file, "tensors": len(out), "bytes": sum(t.numel() * t.element_size() for t in out.values())}


# ------------------------------------------------------------------------------------------------ trellis containers
def migrate_trellis(src: str, dst: str, to: str = "v3", shard_bytes: int = 2 << 30) -> Dict:
    """Rewrite a trellis checkpoint in the other container (``to``: ``"v3"`` sharded with index files, ``"v2"`` layer
    directories).  Quantized parts are copied bit for bit; unquantized tensors follow; side files (config, tokenizer) too."""
    ld = TrellisModelLoader(src)
    weights = {n: ld.load_weight(n) for n in ld.weight_names()}
    part_keys = {tensor_key(n, p, dotted) for n in weights for p in TRELLIS_PARTS for dotted in (False, True)}
    base = {k: ld.load_tensor(k) for k in ld._where if k not in part_keys}
    cfg = None
    if os.path.exists(os.path.join(src, "config.json")):
        with open(os.path.join(src, "config.json")) as f:
            cfg = json.load(f)
    os.makedirs(dst, exist_ok=True)
    if to == "v3":
        save_trellis_v3(weights, base, dst, shard_bytes=shard_bytes, config=cfg)
    elif to == "v2":
        routers = {k: v for k, v in base.items() if ROUTER_PATTERN.search(k)}
        save_trellis_v2(weights, {k: v for k, v in base.items() if k not in routers}, dst, config=cfg, router=routers or None)
    else:
        raise ValueError(to)
    _copy_side_files(src, dst, skip=("config.json",))
    out = TrellisModelLoader(dst)
    return {"from": ld.format, "to": out.format, "weights": len(weights), "base_tensors": len(base), "bits": out.bit_histogram()}


# ------------------------------------------------------------------------------------------------ 2:4 pruning
def prune_checkpoint_24(model_dir: str, out_dir: str, shard_bytes: int = 2 << 30) -> Dict:
    """Magnitude 2:4 pruning of every projection matrix of a float checkpoint (two of every four consecutive input
    weights per output row are zeroed); other tensors are copied.  The result is an ordinary float checkpoint that the
    sparse FP4 layer (``layers.Sparse24Linear``) or any quantizer can take."""
    from .utils.checkpoint import save_checkpoint
    ld = MMFP4ModelLoader(model_dir, prefetch_workers=0)
    out, pruned, kept = {}, 0, 0
    for k in ld.tensor_names():
        t = ld.load_tensor(k)
        if _is_linear_weight(k, ld) and t.shape[1] % 4 == 0:
            g = t.float().reshape(t.shape[0], t.shape[1] // 4, 4)
            keep = torch.zeros_like(g).scatter_(-1, g.abs().topk(2, -1).indices, 1.0)
            out[k] = (g * keep).reshape(t.shape).to(t.dtype)
            pruned += 1
            kept += int((out[k] != 0).sum())
        else:
            out[k] = t
    ld.close()
    os.makedirs(out_dir, exist_ok=True)
    nbytes = sum(t.numel() * t.element_size() for t in out.values())
    files = (save_checkpoint(out, os.path.join(out_dir, "model.safetensors")) if nbytes <= shard_bytes
             else save_checkpoint(out, out_dir, shard_bytes=shard_bytes))
    _copy_side_files(model_dir, out_dir)
    total = sum(out[k].numel() for k in out if _looks_pruned(k, out))
    return {"pruned_matrices": pruned, "files": len(files), "density": round(kept / max(1, total), 4)}


def _looks_pruned(k: str, tensors) -> bool:
    t = tensors[k]
    return k.endswith(".weight") and t.dim() == 2 and not any(s in k for s in ("norm", "embed_tokens", "mlp.gate.weight", "lm_head"))


# ------------------------------------------------------------------------------------------------ draft model
def create_draft_checkpoint(model_dir: str, out_dir: str, num_layers: int = 2, layers: Optional[List[int]] = None) -> Dict:
    """A shallow copy of a checkpoint for speculative decoding: the embeddings, final norm and LM head plus ``num_layers``
    decoder layers (the first ones, or the given ``layers``, renumbered from 0), with ``num_hidden_layers`` (and per-layer
    lists of the configuration) cut to match.  Works on float and on quantized checkpoints alike (tensors are copied as they
    are)."""
    ld = MMFP4ModelLoader(model_dir, prefetch_workers=0)
    pick = list(layers) if layers is not None else list(range(num_layers))
    remap = {old: new for new, old in enumerate(pick)}
    out = {}
    for k in ld.tensor_names():
        li = extract_layer_index(k)
        if li is None:
            out[k] = ld.load_tensor(k)
        elif li in remap:
            out[re.sub(r"(layers\.)%d(\.)" % li, r"\g<1>%d\g<2>" % remap[li], k, count=1)] = ld.load_tensor(k)
    ld.close()
    os.makedirs(out_dir, exist_ok=True)
    save_file(out, os.path.join(out_dir, "model.safetensors"))
    cfg_path = os.path.join(model_dir, "config.json")
    if os.path.exists(cfg_path):
        with open(cfg_path) as f:
            cfg = json.load(f)
        n_old = cfg.get("num_hidden_layers")
        cfg["num_hidden_layers"] = len(pick)
        for key, v in list(cfg.items()):
            if isinstance(v, list) and n_old is not None and len(v) == n_old:
                cfg[key] = [v[i] for i in pick]
        if "first_k_dense_replace" in cfg:
            cfg["first_k_dense_replace"] = sum(1 for i in pick if i < cfg["first_k_dense_replace"])
        with open(os.path.join(out_dir, "config.json"), "w") as f:
            json.dump(cfg, f, indent=1)
    _copy_side_files(model_dir, out_dir, skip=("config.json",))
    return {"layers": pick, "tensors": len(out), "bytes": sum(t.numel() * t.element_size() for t in out.values())}
