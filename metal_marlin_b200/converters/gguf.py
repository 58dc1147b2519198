"""GGUF reader / writer and block de-quantizers.

Parity: reference ``metal_marlin/gguf_loader.py`` (header + metadata + tensor-info parsing, de-quantization of
Q4_0 / Q4_1 / Q5_0 / Q5_1 / Q8_0 / Q2_K / Q4_K / Q5_K / Q6_K / IQ4_NL / IQ4_XS blocks, F16 / BF16 / F32) and ``metal_marlin/gguf_to_marlin.py``
(GGUF -> marlin FP4 incl. MXFP4 blocks with ``e8m0`` scales).  Files are memory-mapped; tensors are de-quantized on
demand with vectorised numpy and can then be re-quantized into this engine's formats.
"""
from __future__ import annotations

import mmap
import struct
from typing import Any, BinaryIO, Dict, List, Optional, Tuple

import numpy as np
import torch

GGUF_MAGIC = 0x46554747      # "GGUF" little endian
# ggml tensor types
F32, F16, Q4_0, Q4_1, Q5_0, Q5_1, Q8_0, Q4_K, Q6_K, BF16, MXFP4 = 0, 1, 2, 3, 6, 7, 8, 12, 14, 30, 39
Q2_K, Q5_K, IQ4_NL, IQ4_XS = 10, 13, 20, 23
TYPE_NAMES = {F32: "F32", F16: "F16", Q4_0: "Q4_0", Q4_1: "Q4_1", Q5_0: "Q5_0", Q5_1: "Q5_1", Q8_0: "Q8_0", Q4_K: "Q4_K",
              Q6_K: "Q6_K", BF16: "BF16", MXFP4: "MXFP4", Q2_K: "Q2_K", Q5_K: "Q5_K", IQ4_NL: "IQ4_NL", IQ4_XS: "IQ4_XS"}
# (elements per block, bytes per block)
BLOCK = {F32: (1, 4), F16: (1, 2), BF16: (1, 2), Q4_0: (32, 18), Q4_1: (32, 20), Q5_0: (32, 22), Q5_1: (32, 24), Q8_0: (32, 34),
         Q4_K: (256, 144), Q6_K: (256, 210), MXFP4: (32, 17), Q2_K: (256, 84), Q5_K: (256, 176), IQ4_NL: (32, 18), IQ4_XS: (256, 136)}
# non-linear 4-bit code book of the IQ4 types
IQ4_VALUES = np.array([-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113], dtype=np.float32)
_VT = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}
E2M1 = np.array([0, 0.5, 1, 1.5, 2, 3, 4, 6, -0.0, -0.5, -1, -1.5, -2, -3, -4, -6], dtype=np.float32)


# ------------------------------------------------------------------------------------------ block de-quantizers
def _f16(b: np.ndarray) -> np.ndarray:
    return b.view(np.float16).astype(np.float32)


def dequant_q4_0(raw: np.ndarray) -> np.ndarray:
    blk = raw.reshape(-1, 18)
    d = _f16(blk[:, :2].copy()).reshape(-1, 1)
    qs = blk[:, 2:]
    q = np.concatenate([qs & 0xF, qs >> 4], 1).astype(np.float32) - 8.0
    return (q * d).reshape(-1)


def dequant_q4_1(raw: np.ndarray) -> np.ndarray:
    blk = raw.reshape(-1, 20)
    d, m = _f16(blk[:, :2].copy()).reshape(-1, 1), _f16(blk[:, 2:4].copy()).reshape(-1, 1)
    qs = blk[:, 4:]
    q = np.concatenate([qs & 0xF, qs >> 4], 1).astype(np.float32)
    return (q * d + m).reshape(-1)


def _q5_high(qh: np.ndarray) -> np.ndarray:
    bits = qh.copy().view(np.uint32).reshape(-1, 1)
    return ((bits >> np.arange(32, dtype=np.uint32)) & 1).astype(np.uint8)      # [n, 32]


def dequant_q5_0(raw: np.ndarray) -> np.ndarray:
    blk = raw.reshape(-1, 22)
    d = _f16(blk[:, :2].copy()).reshape(-1, 1)
    hi = _q5_high(blk[:, 2:6])
    qs = blk[:, 6:]
    lo = np.concatenate([qs & 0xF, qs >> 4], 1)
    return (((lo | (hi << 4)).astype(np.float32) - 16.0) * d).reshape(-1)


def dequant_q5_1(raw: np.ndarray) -> np.ndarray:
    blk = raw.reshape(-1, 24)
    d, m = _f16(blk[:, :2].copy()).reshape(-1, 1), _f16(blk[:, 2:4].copy()).reshape(-1, 1)
    hi = _q5_high(blk[:, 4:8])
    qs = blk[:, 8:]
    lo = np.concatenate([qs & 0xF, qs >> 4], 1)
    return ((lo | (hi << 4)).astype(np.float32) * d + m).reshape(-1)


def dequant_q8_0(raw: np.ndarray) -> np.ndarray:
    blk = raw.reshape(-1, 34)
    d = _f16(blk[:, :2].copy()).reshape(-1, 1)
    return (blk[:, 2:].view(np.int8).astype(np.float32) * d).reshape(-1)


def dequant_q4_k(raw: np.ndarray) -> np.ndarray:
    blk = raw.reshape(-1, 144)
    d, dmin = _f16(blk[:, :2].copy()).reshape(-1, 1), _f16(blk[:, 2:4].copy()).reshape(-1, 1)
    s = blk[:, 4:16].astype(np.uint8)
    sc = np.empty((blk.shape[0], 8), dtype=np.float32)
    mn = np.empty((blk.shape[0], 8), dtype=np.float32)
    for j in range(8):
        if j < 4:
            sc[:, j], mn[:, j] = s[:, j] & 63, s[:, j + 4] & 63
        else:
            sc[:, j] = (s[:, j + 4] & 0xF) | ((s[:, j - 4] >> 6) << 4)
            mn[:, j] = (s[:, j + 4] >> 4) | ((s[:, j] >> 6) << 4)
    qs = blk[:, 16:].reshape(-1, 4, 32)
    lo, hi = (qs & 0xF).astype(np.float32), (qs >> 4).astype(np.float32)
    q = np.stack([lo, hi], 2).reshape(-1, 8, 32)             # sub-blocks 0..7 in order (lo of chunk, hi of chunk)
    return (q * (d * sc)[:, :, None] - (dmin * mn)[:, :, None]).reshape(-1)


def _k_scales(s: np.ndarray):
    """The eight 6-bit (scale, min) pairs packed in the 12 scale bytes of a Q4_K / Q5_K super-block."""
    sc = np.empty((s.shape[0], 8), dtype=np.float32)
    mn = np.empty((s.shape[0], 8), dtype=np.float32)
    for j in range(8):
        if j < 4:
            sc[:, j], mn[:, j] = s[:, j] & 63, s[:, j + 4] & 63
        else:
            sc[:, j] = (s[:, j + 4] & 0xF) | ((s[:, j - 4] >> 6) << 4)
            mn[:, j] = (s[:, j + 4] >> 4) | ((s[:, j] >> 6) << 4)
    return sc, mn


def dequant_q5_k(raw: np.ndarray) -> np.ndarray:
    blk = raw.reshape(-1, 176)
    d, dmin = _f16(blk[:, :2].copy()).reshape(-1, 1), _f16(blk[:, 2:4].copy()).reshape(-1, 1)
    sc, mn = _k_scales(blk[:, 4:16].astype(np.uint8))
    qh = blk[:, 16:48]                                       # bit 2c / 2c + 1 of byte l: fifth bit of chunk c, low / high nibble
    qs = blk[:, 48:].reshape(-1, 4, 32)
    bits = np.stack([(qh >> k) & 1 for k in range(8)], 1).reshape(-1, 4, 2, 32)       # [blk, chunk, lo|hi, l]
    lo = (qs & 0xF) + 16 * bits[:, :, 0]
    hi = (qs >> 4) + 16 * bits[:, :, 1]
    q = np.stack([lo, hi], 2).reshape(-1, 8, 32).astype(np.float32)
    return (q * (d * sc)[:, :, None] - (dmin * mn)[:, :, None]).reshape(-1)


def dequant_q2_k(raw: np.ndarray) -> np.ndarray:
    blk = raw.reshape(-1, 84)
    scales = blk[:, :16]
    qs = blk[:, 16:80].reshape(-1, 2, 32)                    # two halves of 128 elements
    d, dmin = _f16(blk[:, 80:82].copy()).reshape(-1, 1), _f16(blk[:, 82:84].copy()).reshape(-1, 1)
    dl = d * (scales & 0xF).astype(np.float32)               # [blk, 16] sub-blocks of 16 elements
    ml = dmin * (scales >> 4).astype(np.float32)
    # element order inside a half: shift 0: q[0..31], shift 2: q[0..31], ... ; every 16 elements own one (scale, min)
    q = np.stack([(qs >> sh) & 3 for sh in (0, 2, 4, 6)], 2).astype(np.float32)       # [blk, half, shift, 32]
    q = q.reshape(-1, 16, 16)
    return (q * dl[:, :, None] - ml[:, :, None]).reshape(-1)


def dequant_iq4_nl(raw: np.ndarray) -> np.ndarray:
    blk = raw.reshape(-1, 18)
    d = _f16(blk[:, :2].copy()).reshape(-1, 1)
    qs = blk[:, 2:]
    idx = np.concatenate([qs & 0xF, qs >> 4], 1)
    return (IQ4_VALUES[idx] * d).reshape(-1)


def dequant_iq4_xs(raw: np.ndarray) -> np.ndarray:
    blk = raw.reshape(-1, 136)
    d = _f16(blk[:, :2].copy()).reshape(-1, 1)
    sh = blk[:, 2:4].copy().view(np.uint16).astype(np.int32).reshape(-1, 1)
    sl = blk[:, 4:8].astype(np.int32)
    ib = np.arange(8)
    ls = ((sl[:, ib // 2] >> (4 * (ib % 2))) & 0xF) | (((sh >> (2 * ib)) & 3) << 4)     # [blk, 8] 6-bit sub-block scales
    dl = d * (ls - 32).astype(np.float32)
    qs = blk[:, 8:].reshape(-1, 8, 16)
    idx = np.concatenate([qs & 0xF, qs >> 4], 2)             # [blk, 8, 32]
    return (IQ4_VALUES[idx] * dl[:, :, None]).reshape(-1)


def dequant_q6_k(raw: np.ndarray) -> np.ndarray:
    blk = raw.reshape(-1, 210)
    ql, qh = blk[:, :128].reshape(-1, 2, 64), blk[:, 128:192].reshape(-1, 2, 32)
    sc = blk[:, 192:208].view(np.int8).astype(np.float32).reshape(-1, 2, 8)
    d = _f16(blk[:, 208:210].copy()).reshape(-1, 1, 1)
    l0, l1 = ql[:, :, :32], ql[:, :, 32:]
    q1 = ((l0 & 0xF) | ((qh & 3) << 4)).astype(np.int16) - 32
    q2 = ((l1 & 0xF) | (((qh >> 2) & 3) << 4)).astype(np.int16) - 32
    q3 = ((l0 >> 4) | (((qh >> 4) & 3) << 4)).astype(np.int16) - 32
    q4 = ((l1 >> 4) | (((qh >> 6) & 3) << 4)).astype(np.int16) - 32
    q = np.stack([q1, q2, q3, q4], 2).astype(np.float32)    # [n, 2, 4, 32]: y[l], y[l+32], y[l+64], y[l+96]
    isx = np.arange(32) // 16                                # scale index is + {0, 2, 4, 6}
    scale = np.stack([sc[:, :, isx + 0], sc[:, :, isx + 2], sc[:, :, isx + 4], sc[:, :, isx + 6]], 2)    # [n, 2, 4, 32]
    return (q * scale * d[:, :, :, None]).reshape(-1)


def dequant_mxfp4(raw: np.ndarray) -> np.ndarray:
    blk = raw.reshape(-1, 17)
    e = blk[:, 0].astype(np.int32)
    scale = np.ldexp(np.float32(1.0), e - 127).astype(np.float32).reshape(-1, 1)
    qs = blk[:, 1:]
    idx = np.concatenate([qs & 0xF, qs >> 4], 1)
    return (E2M1[idx] * scale).reshape(-1)


_DEQUANT = {Q4_0: dequant_q4_0, Q4_1: dequant_q4_1, Q5_0: dequant_q5_0, Q5_1: dequant_q5_1, Q8_0: dequant_q8_0, Q4_K: dequant_q4_k,
            Q6_K: dequant_q6_k, MXFP4: dequant_mxfp4, Q2_K: dequant_q2_k, Q5_K: dequant_q5_k, IQ4_NL: dequant_iq4_nl,
            IQ4_XS: dequant_iq4_xs}


def dequantize_blocks(raw: np.ndarray, ggml_type: int, n_elements: int) -> np.ndarray:
    if ggml_type == F32:
        return raw.view(np.float32)[:n_elements].astype(np.float32)
    if ggml_type == F16:
        return raw.view(np.float16)[:n_elements].astype(np.float32)
    if ggml_type == BF16:
        return (raw.view(np.uint16)[:n_elements].astype(np.uint32) << 16).view(np.float32)
    try:
        return _DEQUANT[ggml_type](raw)[:n_elements]
    except KeyError:
        raise NotImplementedError(f"GGUF tensor type {ggml_type} is not supported") from None


# ------------------------------------------------------------------------------------------ quantizers (writer side)
def quantize_q8_0(x: np.ndarray) -> np.ndarray:
    b = x.astype(np.float32).reshape(-1, 32)
    d = np.abs(b).max(1, keepdims=True) / 127.0
    q = np.where(d > 0, np.round(b / np.where(d > 0, d, 1)), 0).astype(np.int8)
    return np.concatenate([d.astype(np.float16).view(np.uint8), q.view(np.uint8)], 1).reshape(-1)


def quantize_q4_0(x: np.ndarray) -> np.ndarray:
    b = x.astype(np.float32).reshape(-1, 32)
    idx = np.abs(b).argmax(1)
    mx = b[np.arange(b.shape[0]), idx]
    d = (mx / -8.0).reshape(-1, 1)
    q = np.where(d != 0, np.clip(np.floor(b / np.where(d != 0, d, 1) + 8.5), 0, 15), 8).astype(np.uint8)
    packed = q[:, :16] | (q[:, 16:] << 4)
    return np.concatenate([d.astype(np.float16).view(np.uint8), packed], 1).reshape(-1)


# ------------------------------------------------------------------------------------------ reader
class GGUFReader:
    def __init__(self, path: str):
        self.path = path
        self._f = open(path, "rb")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        self._pos = 0
        magic, self.version = struct.unpack_from("<II", self._mm, 0)
        if magic != GGUF_MAGIC:
            raise ValueError(f"{path} is not a GGUF file")
        if self.version < 2:
            raise ValueError(f"GGUF version {self.version} is not supported (need >= 2)")
        self._pos = 8
        n_tensors, n_kv = self._read("<QQ")
        self.metadata: Dict[str, Any] = {}
        for _ in range(n_kv):
            k = self._string()
            self.metadata[k] = self._value(self._read("<I")[0])
        self.tensors: Dict[str, Tuple[Tuple[int, ...], int, int]] = {}      # name -> (shape (row-major), type, offset)
        for _ in range(n_tensors):
            name = self._string()
            nd = self._read("<I")[0]
            dims = self._read(f"<{nd}Q")
            ttype, off = self._read("<IQ")
            self.tensors[name] = (tuple(reversed(dims)), ttype, off)           # GGUF stores the fastest axis first
        align = int(self.metadata.get("general.alignment", 32))
        self.data_start = (self._pos + align - 1) // align * align

    def _read(self, fmt: str):
        v = struct.unpack_from(fmt, self._mm, self._pos)
        self._pos += struct.calcsize(fmt)
        return v

    def _string(self) -> str:
        n = self._read("<Q")[0]
        s = self._mm[self._pos:self._pos + n].decode("utf-8", errors="replace")
        self._pos += n
        return s

    def _value(self, vt: int):
        if vt == 8:
            return self._string()
        if vt == 9:
            et, n = self._read("<IQ")
            return [self._value(et) for _ in range(n)]
        return self._read(_VT[vt])[0]

    def tensor_names(self) -> List[str]:
        return list(self.tensors)

    def tensor_type(self, name: str) -> str:
        return TYPE_NAMES.get(self.tensors[name][1], str(self.tensors[name][1]))

    def raw(self, name: str) -> np.ndarray:
        shape, ttype, off = self.tensors[name]
        n = int(np.prod(shape))
        be, bb = BLOCK[ttype]
        nbytes = (n + be - 1) // be * bb
        start = self.data_start + off
        return np.frombuffer(self._mm, dtype=np.uint8, count=nbytes, offset=start)

    def load_tensor(self, name: str, dtype=torch.float32) -> torch.Tensor:
        shape, ttype, _ = self.tensors[name]
        n = int(np.prod(shape))
        arr = dequantize_blocks(self.raw(name), ttype, n).reshape(shape)
        return torch.from_numpy(np.ascontiguousarray(arr)).to(dtype)

    def close(self):
        self._mm.close()
        self._f.close()

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()


# ------------------------------------------------------------------------------------------ writer
def _w_string(f: BinaryIO, s: str):
    b = s.encode("utf-8")
    f.write(struct.pack("<Q", len(b)))
    f.write(b)


def write_gguf(path: str, tensors: Dict[str, torch.Tensor], metadata: Optional[Dict[str, Any]] = None,
               types: Optional[Dict[str, int]] = None, alignment: int = 32) -> None:
    """Write float tensors, optionally block-quantizing some (``types[name]`` in F32 / F16 / Q8_0 / Q4_0)."""
    metadata = dict(metadata or {})
    metadata.setdefault("general.alignment", alignment)
    types = types or {}
    blobs, infos, off = [], [], 0
    for name, t in tensors.items():
        tt = types.get(name, F32)
        x = t.detach().to(torch.float32).cpu().numpy()
        if tt == F32:
            raw = x.astype(np.float32).view(np.uint8).reshape(-1)
        elif tt == F16:
            raw = x.astype(np.float16).view(np.uint8).reshape(-1)
        elif tt == Q8_0:
            raw = quantize_q8_0(x)
        elif tt == Q4_0:
            raw = quantize_q4_0(x)
        else:
            raise NotImplementedError(f"writer does not produce type {tt}")
        infos.append((name, tuple(reversed(x.shape)), tt, off))
        blobs.append(raw)
        off = (off + raw.size + alignment - 1) // alignment * alignment
    with open(path, "wb") as f:
        f.write(struct.pack("<IIQQ", GGUF_MAGIC, 3, len(infos), len(metadata)))
        for k, v in metadata.items():
            _w_string(f, k)
            if isinstance(v, str):
                f.write(struct.pack("<I", 8))
                _w_string(f, v)
            elif isinstance(v, bool):
                f.write(struct.pack("<I?", 7, v))
            elif isinstance(v, int):
                f.write(struct.pack("<Iq", 11, v) if v < 0 else struct.pack("<II", 4, v))
            elif isinstance(v, float):
                f.write(struct.pack("<If", 6, v))
            elif isinstance(v, (list, tuple)):
                if all(isinstance(e, str) for e in v):
                    f.write(struct.pack("<IIQ", 9, 8, len(v)))
                    for e in v:
                        _w_string(f, e)
                else:
                    f.write(struct.pack("<IIQ", 9, 5, len(v)))
                    for e in v:
                        f.write(struct.pack("<i", int(e)))
            else:
                raise TypeError(f"unsupported metadata value for {k}: {type(v)}")
        for name, dims, tt, o in infos:
            _w_string(f, name)
            f.write(struct.pack("<I", len(dims)))
            f.write(struct.pack(f"<{len(dims)}Q", *dims))
            f.write(struct.pack("<IQ", tt, o))
        pad = (-f.tell()) % alignment
        f.write(b"\0" * pad)
        for raw in blobs:
            f.write(raw.tobytes())
            f.write(b"\0" * ((-raw.size) % alignment))


# llama.cpp tensor names -> HF names
_GGUF_TO_HF = {
    "token_embd": "model.embed_tokens", "output_norm": "model.norm", "output": "lm_head",
    "attn_q": "self_attn.q_proj", "attn_k": "self_attn.k_proj", "attn_v": "self_attn.v_proj", "attn_output": "self_attn.o_proj",
    "attn_norm": "input_layernorm", "ffn_norm": "post_attention_layernorm", "ffn_gate": "mlp.gate_proj", "ffn_up": "mlp.up_proj",
    "ffn_down": "mlp.down_proj", "attn_q_norm": "self_attn.q_norm", "attn_k_norm": "self_attn.k_norm", "ffn_gate_inp": "mlp.gate",
}


def gguf_name_to_hf(name: str) -> str:
    parts = name.split(".")
    suffix = parts[-1] if parts[-1] in ("weight", "bias") else None
    core = parts[:-1] if suffix else parts
    if core[0] == "blk" and len(core) >= 3:
        mapped = _GGUF_TO_HF.get(core[2], core[2])
        out = f"model.layers.{core[1]}.{mapped}"
    else:
        out = _GGUF_TO_HF.get(core[0], ".".join(core))
    return out + (f".{suffix}" if suffix else "")
