"""``.qmi4`` tensors (asymmetric uint4 with fp16 scales and zero points per group) and the artifact manifest of the
Qwen3.6-27B hybrid: read / write the container, import a directory of prototype tensors into a manifest with raw parts,
validate coverage, and load any artifact as an INT4 layer of this engine.

Container (little endian): ``"QMI4v1\\0\\0"``, then uint32 version (2), in_features, out_features, group_size, packed_k =
ceil(in / 8), groups = ceil(in / group_size), source_out_features, row_begin, row_count, then uint64 byte counts of qweight /
scales / zeros, uint32 key length; then the source key (utf-8), ``qweight`` uint32 ``[packed_k, out]`` (eight codes per word
along the input axis, first code in the low bits), ``scales`` and ``zeros`` fp16 ``[groups, out]``;
``w[k, n] = (code - zero[k / gs, n]) * scale[k / gs, n]``.

Parity: reference ``metal_marlin/qwen36_27b_qmi4.py`` (``read_qmi4_tensor`` ``:84``, ``role_from_legacy_name``, ``write_tensor_parts``,
directory import), ``qwen36_27b_artifact.py`` (roles, ``Int4TensorArtifact`` ``:148``, ``Qwen36ArtifactManifest`` ``:196``,
``write_manifest`` / ``read_manifest``, required-role and full-layer coverage checks) and ``qwen36_27b_profile.py`` (shape
contract; here derived from the ``qwen3.6-27b-hybrid`` preset).  A loaded artifact is a ``layers.QuantizedLinear``: the codes
run on the INT4 weight-streaming kernel for decode and inside the tcgen05 GEMM's main loop for prompts.
"""
from __future__ import annotations

import json
import os
import struct
from dataclasses import asdict, dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..quant.rtn import QuantizedTensor

QMI4_MAGIC = b"QMI4v1\0\0"
QMI4_VERSION = 2
_HEADER = struct.Struct("<8s9I3QI")
SCHEMA_VERSION = "qwen36_27b_int4_v1"
MODEL_ID = "Qwen/Qwen3.6-27B"

LINEAR_ATTENTION_ROLES = ("linear_attn_q", "linear_attn_k", "linear_attn_v", "linear_attn_beta", "linear_attn_a", "linear_attn_z",
                          "linear_attn_out")
FULL_ATTENTION_ROLES = ("full_attn_q", "full_attn_k", "full_attn_v", "full_attn_o")
DENSE_MLP_ROLES = ("mlp_gate", "mlp_up", "mlp_down")
GLOBAL_ROLES = ("lm_head",)
LAYER_ROLES = LINEAR_ATTENTION_ROLES + FULL_ATTENTION_ROLES + DENSE_MLP_ROLES
REQUIRED_ROLES = LAYER_ROLES + GLOBAL_ROLES
LEGACY_NAMES = {"q": "linear_attn_q", "k": "linear_attn_k", "v": "linear_attn_v", "b": "linear_attn_beta", "beta": "linear_attn_beta",
                "a": "linear_attn_a", "z": "linear_attn_z", "out": "linear_attn_out", "attn_q": "full_attn_q", "attn_k": "full_attn_k",
                "attn_v": "full_attn_v", "attn_o": "full_attn_o", "mlp_gate": "mlp_gate", "mlp_up": "mlp_up", "mlp_down": "mlp_down",
                "lm_head": "lm_head"}


def role_shapes(cfg=None) -> Dict[str, Tuple[int, int]]:
    """``role -> (in_features, out_features)`` for a hybrid configuration (default: the ``qwen3.6-27b-hybrid`` preset)."""
    if cfg is None:
        from ..models.config import get_preset
        cfg = get_preset("qwen3.6-27b-hybrid")
    h = cfg.hidden_size
    qk = cfg.linear_num_key_heads * cfg.linear_key_head_dim
    vv = cfg.linear_num_value_heads * cfg.linear_value_head_dim
    hv = cfg.linear_num_value_heads
    aq, akv = cfg.num_attention_heads * cfg.dh, cfg.num_key_value_heads * cfg.dh
    return {"linear_attn_q": (h, qk), "linear_attn_k": (h, qk), "linear_attn_v": (h, vv), "linear_attn_beta": (h, hv),
            "linear_attn_a": (h, hv), "linear_attn_z": (h, vv), "linear_attn_out": (vv, h),
            "full_attn_q": (h, aq), "full_attn_k": (h, akv), "full_attn_v": (h, akv), "full_attn_o": (aq, h),
            "mlp_gate": (h, cfg.intermediate_size), "mlp_up": (h, cfg.intermediate_size), "mlp_down": (cfg.intermediate_size, h),
            "lm_head": (h, cfg.vocab_size)}


def expected_tensor_shape(role: str, cfg=None) -> Tuple[int, int]:
    return role_shapes(cfg)[role]


def role_from_legacy_name(name: str) -> str:
    stem = os.path.splitext(os.path.basename(name))[0]
    if stem not in LEGACY_NAMES:
        raise ValueError(f"unsupported tensor name: {name}")
    return LEGACY_NAMES[stem]


# ------------------------------------------------------------------------------------------------ the container
@dataclass
class Qmi4Tensor:
    source_key: str
    in_features: int
    out_features: int
    group_size: int
    qweight: torch.Tensor            # int32 [ceil(in / 8), out]
    scales: torch.Tensor             # fp16 [groups, out]
    zeros: torch.Tensor              # fp16 [groups, out]
    source_out_features: int = 0
    row_begin: int = 0
    row_count: int = 0

    @property
    def packed_k(self) -> int:
        return (self.in_features + 7) // 8

    @property
    def groups(self) -> int:
        return (self.in_features + self.group_size - 1) // self.group_size

    def validate(self) -> None:
        if self.group_size <= 0 or self.group_size % 8:
            raise ValueError(f"group_size must be a positive multiple of 8, got {self.group_size}")
        if tuple(self.qweight.shape) != (self.packed_k, self.out_features):
            raise ValueError(f"qweight shape {tuple(self.qweight.shape)} != {(self.packed_k, self.out_features)}")
        for name, t in (("scales", self.scales), ("zeros", self.zeros)):
            if tuple(t.shape) != (self.groups, self.out_features):
                raise ValueError(f"{name} shape {tuple(t.shape)} != {(self.groups, self.out_features)}")

    def codes(self) -> torch.Tensor:
        """uint8 ``[out, in]``."""
        w = self.qweight.to(torch.int64) & 0xFFFFFFFF
        nib = (w.unsqueeze(1) >> (torch.arange(8, dtype=torch.int64).view(1, 8, 1) * 4)) & 0xF      # [packed_k, 8, out]
        return nib.reshape(self.packed_k * 8, self.out_features)[: self.in_features].t().contiguous().to(torch.uint8)

    def dequantize(self) -> torch.Tensor:
        """fp32 ``[out, in]``."""
        g = torch.arange(self.in_features) // self.group_size
        return (self.codes().float() - self.zeros.float().t()[:, g]) * self.scales.float().t()[:, g]

    def to_linear(self, device=None, bias=None):
        """An INT4 ``QuantizedLinear`` over the same codes, scales and zero points (``in_features`` a multiple of the group)."""
        from ..layers.linear import QuantizedLinear
        if self.in_features % self.group_size:
            raise ValueError("the INT4 kernels need in_features to be a multiple of the group size")
        q = QuantizedTensor(self.codes(), self.scales.t().contiguous(), self.zeros.t().contiguous(), "int4", self.group_size, 4)
        return QuantizedLinear(q, bias, device)


def quantize_to_qmi4(w: torch.Tensor, group_size: int = 128, source_key: str = "") -> Qmi4Tensor:
    """Asymmetric uint4 round-to-nearest of ``w [out, in]``: per group ``scale = (max - min) / 15``, ``zero = -min / scale``."""
    out_f, in_f = w.shape
    if in_f % group_size or in_f % 8:
        raise ValueError("in_features must be a multiple of the group size and of 8")
    g = w.detach().float().view(out_f, in_f // group_size, group_size)
    lo, hi = g.amin(-1, keepdim=True), g.amax(-1, keepdim=True)
    scale = ((hi - lo) / 15.0).clamp_min(1e-8).to(torch.float16).float()
    zero = (-lo / scale).round().clamp_(0, 15)
    codes = (g / scale + zero).round().clamp_(0, 15).to(torch.int64).view(out_f, in_f)
    words = (codes.t().reshape(in_f // 8, 8, out_f) << (torch.arange(8).view(1, 8, 1) * 4)).sum(1)
    words = torch.where(words >= 2 ** 31, words - 2 ** 32, words).to(torch.int32)
    return Qmi4Tensor(source_key, in_f, out_f, group_size, words, scale.squeeze(-1).t().contiguous().to(torch.float16),
                      zero.squeeze(-1).t().contiguous().to(torch.float16), out_f, 0, out_f)


def write_qmi4_tensor(path: str, t: Qmi4Tensor) -> None:
    t.validate()
    key = t.source_key.encode("utf-8")
    qb = t.qweight.contiguous().numpy().astype("<i4").tobytes()
    sb = t.scales.contiguous().numpy().astype("<f2").tobytes()
    zb = t.zeros.contiguous().numpy().astype("<f2").tobytes()
    head = _HEADER.pack(QMI4_MAGIC, QMI4_VERSION, t.in_features, t.out_features, t.group_size, t.packed_k, t.groups,
                        t.source_out_features or t.out_features, t.row_begin, t.row_count or t.out_features, len(qb), len(sb), len(zb),
                        len(key))
    with open(path, "wb") as f:
        f.write(head + key + qb + sb + zb)


def read_qmi4_tensor(path: str) -> Qmi4Tensor:
    data = open(path, "rb").read()
    if len(data) < _HEADER.size:
        raise ValueError(f"{path} is too small to be a qmi4 tensor")
    (magic, version, in_f, out_f, gs, packed_k, groups, src_out, row_begin, row_count, qn, sn, zn, key_len) = _HEADER.unpack_from(data)
    if magic != QMI4_MAGIC:
        raise ValueError(f"{path}: not a qmi4 tensor (magic {magic!r})")
    if version != QMI4_VERSION:
        raise ValueError(f"{path}: unsupported qmi4 version {version}")
    o = _HEADER.size
    ends = [o + key_len, o + key_len + qn, o + key_len + qn + sn, o + key_len + qn + sn + zn]
    if ends[-1] != len(data):
        raise ValueError(f"{path}: the header describes {ends[-1]} bytes, the file has {len(data)}")
    if qn != packed_k * out_f * 4 or sn != groups * out_f * 2 or zn != sn:
        raise ValueError(f"{path}: section sizes do not match the dimensions")
    key = data[o: ends[0]].decode("utf-8")
    qw = torch.from_numpy(np.frombuffer(data, "<i4", packed_k * out_f, ends[0]).reshape(packed_k, out_f).copy())
    sc = torch.from_numpy(np.frombuffer(data, "<f2", groups * out_f, ends[1]).reshape(groups, out_f).copy())
    zp = torch.from_numpy(np.frombuffer(data, "<f2", groups * out_f, ends[2]).reshape(groups, out_f).copy())
    t = Qmi4Tensor(key, in_f, out_f, gs, qw, sc, zp, src_out, row_begin, row_count)
    if t.packed_k != packed_k or t.groups != groups:
        raise ValueError(f"{path}: packed_k / groups do not follow from in_features and group_size")
    t.validate()
    return t


# ------------------------------------------------------------------------------------------------ the manifest
@dataclass
class Int4TensorArtifact:
    role: str
    layer_index: Optional[int]
    qweight: str                     # raw files, relative to the manifest
    scales: str
    zeros: str
    in_features: int
    out_features: int
    group_size: int = 128
    dtype: str = "uint4_asym"
    qweight_layout: str = "packed_k_major_u32"
    metadata_layout: str = "group_major_f16"
    calibration: Dict[str, Any] = field(default_factory=dict)

    def validate(self, shapes: Optional[Dict[str, Tuple[int, int]]] = None) -> None:
        shapes = shapes or role_shapes()
        if self.role not in shapes:
            raise ValueError(f"unsupported tensor role: {self.role}")
        if (self.in_features, self.out_features) != shapes[self.role]:
            raise ValueError(f"{self.role} expected shape {shapes[self.role]}, got {(self.in_features, self.out_features)}")
        if self.in_features % 8:
            raise ValueError("the packed layout needs in_features divisible by 8")
        if self.group_size <= 0 or self.group_size % 8:
            raise ValueError("group_size must be a positive multiple of 8")
        if self.layer_index is None and self.role not in GLOBAL_ROLES + LAYER_ROLES:
            raise ValueError(f"{self.role}: unknown role")


@dataclass
class ArtifactManifest:
    tensors: List[Int4TensorArtifact]
    schema_version: str = SCHEMA_VERSION
    model_id: str = MODEL_ID
    source_checkpoint: str = MODEL_ID
    notes: str = "Qwen3.6-27B dense hybrid artifact"

    def validate(self, shapes=None) -> None:
        if self.schema_version != SCHEMA_VERSION:
            raise ValueError(f"unsupported schema_version: {self.schema_version}")
        shapes = shapes or role_shapes()
        seen = set()
        for t in self.tensors:
            t.validate(shapes)
            key = (t.layer_index, t.role)
            if key in seen:
                raise ValueError(f"duplicate artifact for layer {t.layer_index} role {t.role}")
            seen.add(key)

    def index(self) -> Dict[Tuple[Optional[int], str], Int4TensorArtifact]:
        return {(t.layer_index, t.role): t for t in self.tensors}


def write_manifest(manifest: ArtifactManifest, path: str, shapes=None) -> str:
    manifest.validate(shapes)
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    with open(path, "w", encoding="utf-8") as f:
        f.write(json.dumps(asdict(manifest), indent=2, sort_keys=True) + "\n")
    return path


def read_manifest(path: str, shapes=None) -> ArtifactManifest:
    with open(path, encoding="utf-8") as f:
        d = json.load(f)
    m = ArtifactManifest([Int4TensorArtifact(**t) for t in d.get("tensors", [])], d.get("schema_version", SCHEMA_VERSION),
                         d.get("model_id", MODEL_ID), d.get("source_checkpoint", MODEL_ID), d.get("notes", ""))
    m.validate(shapes)
    return m


def layer_roles(cfg, layer: int) -> Tuple[str, ...]:
    """Roles a concrete layer needs: its mixer (linear or full attention) and the dense MLP."""
    return (LINEAR_ATTENTION_ROLES if cfg.layer_is_linear(layer) else FULL_ATTENTION_ROLES) + DENSE_MLP_ROLES


def validate_required_roles(manifest: ArtifactManifest, roles: Sequence[str] = REQUIRED_ROLES, shapes=None) -> None:
    """A template manifest: exactly one artifact per role (layer index ``None``)."""
    manifest.validate(shapes)
    have = [t.role for t in manifest.tensors]
    missing = [r for r in roles if have.count(r) == 0]
    dup = [r for r in roles if have.count(r) > 1]
    if missing or dup:
        raise ValueError(f"manifest roles: missing {missing}, duplicated {dup}")


def validate_full_layer_coverage(manifest: ArtifactManifest, cfg=None, shapes=None) -> None:
    """Every concrete layer has the roles of its kind, the global tensors exist, and no template entry is left."""
    if cfg is None:
        from ..models.config import get_preset
        cfg = get_preset("qwen3.6-27b-hybrid")
    manifest.validate(shapes or role_shapes(cfg))
    idx = manifest.index()
    stray = sorted(r for (li, r) in idx if li is None and r in LAYER_ROLES)
    if stray:
        raise ValueError(f"template (layer-less) entries in a full-layer manifest: {stray}")
    problems = []
    for li in range(cfg.num_hidden_layers):
        miss = [r for r in layer_roles(cfg, li) if (li, r) not in idx]
        if miss:
            problems.append(f"layer {li}: {miss}")
    problems += [f"global: {r}" for r in GLOBAL_ROLES if (None, r) not in idx]
    if problems:
        raise ValueError("incomplete coverage: " + "; ".join(problems[:8]) + (" ..." if len(problems) > 8 else ""))


def write_tensor_parts(t: Qmi4Tensor, out_dir: str, prefix: str) -> Tuple[str, str, str]:
    os.makedirs(out_dir, exist_ok=True)
    names = (f"{prefix}.qweight.u32.bin", f"{prefix}.scales.f16.bin", f"{prefix}.zeros.f16.bin")
    for name, arr, dt in zip(names, (t.qweight, t.scales, t.zeros), ("<i4", "<f2", "<f2")):
        with open(os.path.join(out_dir, name), "wb") as f:
            f.write(arr.contiguous().numpy().astype(dt).tobytes())
    return names


def import_qmi4_directory(src_dir: str, out_dir: str, layer_index: Optional[int] = None, cfg=None, shapes=None) -> ArtifactManifest:
    """Turn a directory of prototype ``<name>.qmi4`` files (``q.qmi4``, ``attn_o.qmi4``, ``mlp_down.qmi4`` ...) into raw parts
    plus ``manifest.json`` in ``out_dir``; ``layer_index`` ``None`` writes a template manifest."""
    shapes = shapes or role_shapes(cfg)
    arts = []
    for fname in sorted(os.listdir(src_dir)):
        if not fname.endswith(".qmi4"):
            continue
        role = role_from_legacy_name(fname)
        t = read_qmi4_tensor(os.path.join(src_dir, fname))
        li = None if role in GLOBAL_ROLES else layer_index
        prefix = role if li is None else f"layer{li:03d}.{role}"
        qn, sn, zn = write_tensor_parts(t, out_dir, prefix)
        arts.append(Int4TensorArtifact(role, li, qn, sn, zn, t.in_features, t.out_features, t.group_size,
                                       calibration={"source_tensor": t.source_key, "source_qmi4": fname, "row_begin": t.row_begin,
                                                    "row_count": t.row_count, "source_out_features": t.source_out_features}))
    m = ArtifactManifest(arts)
    write_manifest(m, os.path.join(out_dir, "manifest.json"), shapes)
    return m


def load_artifact(manifest_dir: str, art: Int4TensorArtifact) -> Qmi4Tensor:
    """Read the raw parts of one manifest entry back into a tensor record."""
    pk, g = (art.in_features + 7) // 8, (art.in_features + art.group_size - 1) // art.group_size

    def raw(name, dt, shape):
        return torch.from_numpy(np.fromfile(os.path.join(manifest_dir, name), dtype=dt).reshape(shape).copy())
    t = Qmi4Tensor(art.calibration.get("source_tensor", art.role), art.in_features, art.out_features, art.group_size,
                   raw(art.qweight, "<i4", (pk, art.out_features)), raw(art.scales, "<f2", (g, art.out_features)),
                   raw(art.zeros, "<f2", (g, art.out_features)))
    t.validate()
    return t


def load_layer_linears(manifest_dir: str, layer: Optional[int], device=None, shapes=None) -> Dict[str, Any]:
    """``role -> QuantizedLinear`` for the entries of one layer (``None``: the template / global entries)."""
    m = read_manifest(os.path.join(manifest_dir, "manifest.json"), shapes)
    return {t.role: load_artifact(manifest_dir, t).to_linear(device) for t in m.tensors if t.layer_index == layer}
