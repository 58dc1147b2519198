"""Trellis (v2 layer directories / v3 HF shards) checkpoint format: codebook, tile packing, loader, writer.

Per quantized weight ``W [out, in]`` four tensors keyed ``name.replace('.', '__') + {__indices, __scales, __su, __sv}``
(v3 also allows dotted ``.indices/.scales/.su/.sv``):

* ``indices uint8 [1 + tiles_out * tiles_in * ceil(256 * bits / 8)]`` — byte 0 is ``bits`` (2..8); then 16x16
  tiles in ``[tile_out][tile_in]`` order, each a little-endian, LSB-first bitstream of 256 codes with code index
  ``local_out * 16 + local_in``;
* ``scales fp32 [ceil(in / gs), out]``; ``su fp32 [in]``; ``sv fp32 [out]`` (both +-1).

Dequantization: ``W[o, i] = grid_bits[code] * scales[i // gs, o] * sv[o] * su[i]`` with the uniform grid
``linspace(-(2^b - 1) / 2, (2^b - 1) / 2, 2^b) * 1.24371088``.

Parity: reference ``metal_marlin/trellis/loader.py:50-110,156,551-660`` (formats, ``TrellisWeight``, legacy int16
rejection ``:623-627``), ``metal_marlin/trellis/linear.py:533-610`` (dequantization rule, su/sv role swap),
``metal_marlin/quantization/trellis_codebook.py:18-57`` (grid), ``metal_marlin/trellis/packing.py`` and
``metal_marlin/trellis/shard_writer.py`` (writers), packer ``scripts/quantize_glm47_flash_cuda.py:108-262``.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Sequence, Dict, Iterable, List, Optional, Tuple

import torch

from .safetensors_io import SafetensorsFile, save_file

GRID_SCALE = 1.24371088
TILE = 16


def trellis_grid(bits: int, device="cpu", dtype=torch.float32) -> torch.Tensor:
    n = 1 << bits
    half = (n - 1) / 2.0
    return torch.linspace(-half, half, n, device=device, dtype=torch.float32).mul_(GRID_SCALE).to(dtype)


def tile_bytes(bits: int) -> int:
    return (256 * bits + 7) // 8


def pack_codes(codes: torch.Tensor, bits: int) -> torch.Tensor:
    """``codes uint8 [out, in]`` -> ``uint8 [1 + tiles_out * tiles_in * tile_bytes]`` (header byte included).
    Ragged edges are padded with code 0."""
    out_f, in_f = codes.shape
    to, ti = -(-out_f // TILE), -(-in_f // TILE)
    c = torch.zeros(to * TILE, ti * TILE, dtype=torch.int64, device=codes.device)
    c[:out_f, :in_f] = codes.to(torch.int64)
    tiles = c.view(to, TILE, ti, TILE).permute(0, 2, 1, 3).reshape(to * ti, 256)
    bitpos = torch.arange(bits, device=codes.device)
    stream = ((tiles.unsqueeze(-1) >> bitpos) & 1).reshape(to * ti, 256 * bits)
    pad = tile_bytes(bits) * 8 - 256 * bits
    if pad:
        stream = torch.cat([stream, torch.zeros(to * ti, pad, dtype=stream.dtype, device=stream.device)], 1)
    by = (stream.view(to * ti, -1, 8) << torch.arange(8, device=codes.device)).sum(-1).to(torch.uint8)
    return torch.cat([torch.tensor([bits], dtype=torch.uint8, device=codes.device), by.reshape(-1)])


def unpack_codes(indices: torch.Tensor, out_f: int, in_f: int) -> Tuple[torch.Tensor, int]:
    """Inverse of :func:`pack_codes`; returns (codes uint8 [out, in], bits)."""
    if indices.dtype not in (torch.uint8,):
        raise ValueError(f"unsupported trellis index dtype {indices.dtype} (legacy int16 indices are not supported)")
    flat = indices.reshape(-1)
    bits = int(flat[0])
    if not 2 <= bits <= 8:
        raise ValueError(f"invalid trellis bit width {bits}")
    to, ti = -(-out_f // TILE), -(-in_f // TILE)
    tb = tile_bytes(bits)
    body = flat[1:1 + to * ti * tb]
    if body.numel() != to * ti * tb:
        raise ValueError(f"index blob has {flat.numel() - 1} bytes, expected {to * ti * tb}")
    by = body.view(to * ti, tb).to(torch.int64)
    stream = ((by.unsqueeze(-1) >> torch.arange(8, device=by.device)) & 1).reshape(to * ti, tb * 8)[:, :256 * bits]
    codes = (stream.view(to * ti, 256, bits) << torch.arange(bits, device=by.device)).sum(-1)
    codes = codes.view(to, ti, TILE, TILE).permute(0, 2, 1, 3).reshape(to * TILE, ti * TILE)
    return codes[:out_f, :in_f].to(torch.uint8).contiguous(), bits


@dataclass
class TrellisWeight:
    """One quantized matrix in checkpoint form."""
    indices: torch.Tensor            # uint8 blob with header byte
    scales: torch.Tensor             # fp32 [n_groups, out]
    su: torch.Tensor                 # fp32 [in]
    sv: torch.Tensor                 # fp32 [out]
    shape: Tuple[int, int]           # (out, in)
    name: str = ""

    @property
    def bits(self) -> int:
        return int(self.indices.reshape(-1)[0])

    @property
    def group_size(self) -> int:
        return -(-self.shape[1] // self.scales.shape[0])

    def codes(self) -> torch.Tensor:
        return unpack_codes(self.indices, *self.shape)[0]

    def dequantize(self, dtype=torch.float32) -> torch.Tensor:
        out_f, in_f = self.shape
        codes, bits = unpack_codes(self.indices, out_f, in_f)
        grid = trellis_grid(bits, codes.device)
        su, sv = self.su.float(), self.sv.float()
        if su.numel() == out_f and sv.numel() == in_f and out_f != in_f:
            su, sv = sv, su                                    # roles swapped by some writers
        gs = self.group_size
        g_idx = (torch.arange(in_f, device=codes.device) // gs).clamp_(max=self.scales.shape[0] - 1)
        sc = self.scales.float()[g_idx, :].t()                 # [out, in]
        return (grid[codes.long()] * sc * sv.view(-1, 1) * su.view(1, -1)).to(dtype)


def quantize_trellis(w: torch.Tensor, bits: int, group_size: int = 128, seed: int = 0, random_signs: bool = True) -> TrellisWeight:
    """Nearest-grid quantizer producing the trellis container (the reference's "Viterbi" search reduces to
    nearest-neighbour on this uniform scalar grid).  ``su``/``sv`` are random sign flips (a diagonal +-1
    rotation) as written by the reference's quantizer."""
    out_f, in_f = w.shape
    g = torch.Generator(device="cpu").manual_seed(seed)
    if random_signs:
        su = (torch.randint(0, 2, (in_f,), generator=g).float() * 2 - 1).to(w.device)
        sv = (torch.randint(0, 2, (out_f,), generator=g).float() * 2 - 1).to(w.device)
    else:
        su, sv = torch.ones(in_f, device=w.device), torch.ones(out_f, device=w.device)
    wr = w.float() * sv.view(-1, 1) * su.view(1, -1)
    ng = -(-in_f // group_size)
    pad = ng * group_size - in_f
    wp = torch.nn.functional.pad(wr, (0, pad)) if pad else wr
    grp = wp.view(out_f, ng, group_size)
    gmax = (((1 << bits) - 1) / 2.0) * GRID_SCALE
    scale = (grp.abs().amax(-1) / gmax).clamp_min(1e-12)      # [out, ng]
    half = ((1 << bits) - 1) / 2.0
    codes = ((grp / scale.unsqueeze(-1)) / GRID_SCALE + half).round().clamp_(0, (1 << bits) - 1)
    codes = codes.view(out_f, ng * group_size)[:, :in_f].to(torch.uint8)
    return TrellisWeight(pack_codes(codes, bits).cpu(), scale.t().contiguous().float().cpu(), su.cpu(), sv.cpu(), (out_f, in_f))


# ---------------------------------------------------------------------------------------------
# containers
# ---------------------------------------------------------------------------------------------
SUFFIXES = ("indices", "scales", "su", "sv")


def tensor_key(name: str, part: str, dotted: bool = False) -> str:
    return f"{name}.{part}" if dotted else name.replace(".", "__") + "__" + part


def detect_trellis_format(path: str) -> Optional[str]:
    if os.path.exists(os.path.join(path, "quantization_index.json")) and \
            os.path.exists(os.path.join(path, "model.safetensors.index.json")):
        return "v3_hf_shards"
    if os.path.isdir(os.path.join(path, "layer_0000")):
        return "v2_layers"
    return None


def save_trellis_v3(weights: Dict[str, TrellisWeight], base: Dict[str, torch.Tensor], out_dir: str,
                    shard_bytes: int = 2 << 30, config: Optional[dict] = None) -> None:
    """HF-shard container: quantized parts + unquantized tensors in shards, ``model.safetensors.index.json``,
    ``quantization_index.json {"layers": [{name, bits, shape, mse}]}``."""
    os.makedirs(out_dir, exist_ok=True)
    items: List[Tuple[str, torch.Tensor]] = []
    qindex = []
    for name, tw in weights.items():
        for part in SUFFIXES:
            items.append((tensor_key(name, part), getattr(tw, part)))
        qindex.append({"name": name, "bits": tw.bits, "shape": list(tw.shape), "mse": 0.0})
    items.extend(base.items())
    weight_map, shard, size, no = {}, {}, 0, 1

    def flush():
        nonlocal shard, size, no
        if shard:
            fn = f"model-{no:05d}.safetensors"
            save_file(shard, os.path.join(out_dir, fn), metadata={"format": "trellis_v3"})
            weight_map.update({k: fn for k in shard})
            shard, size, no = {}, 0, no + 1

    for k, v in items:
        shard[k] = v
        size += v.numel() * v.element_size()
        if size >= shard_bytes:
            flush()
    flush()
    with open(os.path.join(out_dir, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {"format": "trellis_v3"}, "weight_map": weight_map}, f)
    with open(os.path.join(out_dir, "quantization_index.json"), "w") as f:
        json.dump({"layers": qindex}, f)
    if config is not None:
        with open(os.path.join(out_dir, "config.json"), "w") as f:
            json.dump(config, f, indent=1)


def save_trellis_v2(weights: Dict[str, TrellisWeight], base: Dict[str, torch.Tensor], out_dir: str,
                    config: Optional[dict] = None, router: Optional[Dict[str, torch.Tensor]] = None) -> None:
    """Layer-directory container: ``layer_NNNN/index.json`` + ``tensor_*.safetensors``, ``base_weights.safetensors``,
    optional ``router_weights.safetensors``.  Weights that belong to no layer go to ``layer_0000``."""
    from .mmfp4_loader import extract_layer_index
    os.makedirs(out_dir, exist_ok=True)
    per_layer: Dict[int, Dict[str, TrellisWeight]] = {}
    for name, tw in weights.items():
        per_layer.setdefault(extract_layer_index(name) or 0, {})[name] = tw
    for li, ws in per_layer.items():
        d = os.path.join(out_dir, f"layer_{li:04d}")
        os.makedirs(d, exist_ok=True)
        entries = []
        for j, (name, tw) in enumerate(ws.items()):
            save_file({tensor_key(name, p): getattr(tw, p) for p in SUFFIXES}, os.path.join(d, f"tensor_{j:04d}.safetensors"))
            entries.append({"name": name, "bits": tw.bits, "shape": list(tw.shape), "mse": 0.0})
        with open(os.path.join(d, "index.json"), "w") as f:
            json.dump({"tensors": entries}, f)
    save_file(base, os.path.join(out_dir, "base_weights.safetensors"))
    if router:
        save_file(router, os.path.join(out_dir, "router_weights.safetensors"))
    if config is not None:
        with open(os.path.join(out_dir, "config.json"), "w") as f:
            json.dump(config, f, indent=1)


class TrellisModelLoader:
    """Uniform access to both containers."""

    def __init__(self, path: str):
        self.path = path
        self.format = detect_trellis_format(path)
        if self.format is None:
            raise FileNotFoundError(f"{path} is not a trellis checkpoint (no quantization_index.json / layer_0000)")
        self.meta: Dict[str, dict] = {}          # weight name -> {bits, shape}
        self._where: Dict[str, str] = {}         # tensor key -> file
        self._base_files: List[str] = []
        if self.format == "v3_hf_shards":
            with open(os.path.join(path, "quantization_index.json")) as f:
                for e in json.load(f)["layers"]:
                    self.meta[e["name"]] = e
            with open(os.path.join(path, "model.safetensors.index.json")) as f:
                self._where = {k: os.path.join(path, v) for k, v in json.load(f)["weight_map"].items()}
            bw = os.path.join(path, "base_weights.safetensors")
            if os.path.exists(bw):
                self._base_files.append(bw)
        else:
            for d in sorted(x for x in os.listdir(path) if x.startswith("layer_")):
                ld = os.path.join(path, d)
                with open(os.path.join(ld, "index.json")) as f:
                    for e in json.load(f)["tensors"]:
                        self.meta[e["name"]] = e
                for fn in sorted(os.listdir(ld)):
                    if fn.endswith(".safetensors"):
                        with SafetensorsFile(os.path.join(ld, fn)) as sf:
                            for k in sf.keys():
                                self._where[k] = os.path.join(ld, fn)
            for fn in ("base_weights.safetensors", "router_weights.safetensors"):
                if os.path.exists(os.path.join(path, fn)):
                    self._base_files.append(os.path.join(path, fn))
        for bf in self._base_files:
            with SafetensorsFile(bf) as sf:
                for k in sf.keys():
                    self._where.setdefault(k, bf)

    def weight_names(self) -> List[str]:
        return list(self.meta.keys())

    def has_weight(self, name: str) -> bool:
        return name in self.meta

    def _get(self, key: str) -> torch.Tensor:
        with SafetensorsFile(self._where[key]) as sf:
            return sf.get_tensor(key)

    def load_weight(self, name: str) -> TrellisWeight:
        e = self.meta[name]
        parts = {}
        for p in SUFFIXES:
            k = tensor_key(name, p)
            if k not in self._where:
                k = tensor_key(name, p, dotted=True)
            parts[p] = self._get(k)
        if parts["indices"].dtype == torch.int16:
            raise ValueError(f"{name}: legacy int16 trellis indices are not supported; re-quantize the checkpoint")
        return TrellisWeight(parts["indices"], parts["scales"].float(), parts["su"].float(), parts["sv"].float(),
                             tuple(e["shape"]), name)

    def has_tensor(self, name: str) -> bool:
        return name in self._where

    def load_tensor(self, name: str) -> torch.Tensor:
        return self._get(name)

    def bit_histogram(self) -> Dict[int, int]:
        h: Dict[int, int] = {}
        for e in self.meta.values():
            h[e["bits"]] = h.get(e["bits"], 0) + 1
        return dict(sorted(h.items()))


def quantize_model_trellis(model_dir: str, out_dir: str, bits: int = 4, group_size: int = 128, device: str = "cpu",
                           container: str = "v3", bit_allocation: Optional[Dict[str, int]] = None,
                           hessians: Optional[Dict[str, torch.Tensor]] = None, target_bpw: Optional[float] = None,
                           bit_choices: Sequence[int] = (2, 3, 4, 5, 6, 8)) -> dict:
    """Quantize a float HF checkpoint into a trellis container.  Linear weights (2-D, not embeddings / norms /
    routers) become trellis tensors at ``bits`` (or ``bit_allocation[name]``); everything else is kept as is.

    ``hessians`` (``name -> X^T X`` of the layer's inputs): matrices that have one are quantized with LDL error feedback
    (``quant/ldlq.py``) instead of plain nearest-grid rounding.  ``target_bpw``: mixed bit widths - every matrix is tried at
    each of ``bit_choices``, its error on the Hessian metric (plain squared error without a Hessian) recorded, and bits are
    handed out greedily by error drop per byte until the average reaches the target (``quant.mixed_precision.allocate_bits``)."""
    from ..quant.convert import iter_safetensors_weights, should_quantize_tensor
    weights: Dict[str, TrellisWeight] = {}
    base: Dict[str, torch.Tensor] = {}
    errs = []
    hessians = hessians or {}

    def usable(name, t):
        H = hessians.get(name)
        gs = group_size if t.shape[1] % group_size == 0 else 16
        return H if (H is not None and t.shape[1] % 16 == 0 and H.shape[0] == t.shape[1]) else None, gs

    if target_bpw is not None and bit_allocation is None:
        from ..quant.ldlq import proxy_error
        from ..quant.mixed_precision import allocate_bits
        sens, sizes = {}, {}
        for name, t in iter_safetensors_weights(model_dir):
            if not should_quantize_tensor(name, t):
                continue
            w = t.to(device=device, dtype=torch.float32)
            H, gs = usable(name, t)
            sizes[name] = w.numel()
            sens[name] = {}
            for b in bit_choices:
                dq = quantize_trellis(w, b, gs, random_signs=False).dequantize().to(w.device)
                # absolute (not relative) error, so that large and sensitive matrices attract the bits
                sens[name][b] = (proxy_error(w, dq, H.to(w.device)) * float(torch.einsum("oi,ij,oj->", w.double(), H.to(w.device).double(), w.double()))
                                 if H is not None else float((w - dq).pow(2).sum()))
        bit_allocation = allocate_bits(sens, sizes, target_bpw, bit_choices)
    n_ldlq = 0
    for name, t in iter_safetensors_weights(model_dir):
        if should_quantize_tensor(name, t):
            b = (bit_allocation or {}).get(name, bits)
            H, gs = usable(name, t)
            if H is not None:
                from ..quant.ldlq import ldlq_quantize
                tw = ldlq_quantize(t.to(device=device, dtype=torch.float32), H.to(device), b, gs, seed=len(weights)).weight
                n_ldlq += 1
            else:
                tw = quantize_trellis(t.to(device=device, dtype=torch.float32), b, group_size, seed=len(weights))
            tw.name = name
            weights[name] = tw
            w = t.float()
            errs.append(float((tw.dequantize().to(w.device) - w).pow(2).mean().sqrt() / w.pow(2).mean().sqrt().clamp_min(1e-12)))
        else:
            base[name] = t
    cfg = None
    cp = os.path.join(model_dir, "config.json")
    if os.path.exists(cp):
        with open(cp) as f:
            cfg = json.load(f)
        cfg["quantization_config"] = {"format": "trellis_" + container, "bits": bits, "group_size": group_size}
    (save_trellis_v3 if container == "v3" else save_trellis_v2)(weights, base, out_dir, config=cfg)
    for fn in ("tokenizer.json", "tokenizer_config.json", "generation_config.json", "special_tokens_map.json"):
        if os.path.exists(os.path.join(model_dir, fn)):
            import shutil
            shutil.copy(os.path.join(model_dir, fn), os.path.join(out_dir, fn))
    n_w = sum(tw.shape[0] * tw.shape[1] for tw in weights.values())
    return {"quantized": len(weights), "tensors": len(weights) + len(base), "bits": bits, "ldlq": n_ldlq,
            "mean_bpw": sum(tw.shape[0] * tw.shape[1] * tw.bits for tw in weights.values()) / max(1, n_w),
            "mean_rel_rmse": sum(errs) / max(1, len(errs)), "format": "trellis_" + container}
