"""Dependency-free safetensors reader/writer.

The container is an 8-byte little-endian header length, a JSON header mapping
tensor name -> {dtype, shape, data_offsets}, then raw little-endian data.
Parity: reference ``metal_marlin/mmfp4_loader.py:521`` (``_read_safetensors_header``)
parses the same header by hand; ``metal_marlin/mmap_loader.py`` memory-maps it.

The reader memory-maps the file so a 100+ GB sharded checkpoint can be walked
tensor by tensor; ``uint32``/``uint16`` (which torch lacks as first-class dtypes)
are returned as ``int32``/``int16`` views with identical bits.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, Iterator, Mapping, Optional, Tuple

import numpy as np
import torch

_ST2NP = {
    "F64": np.float64, "F32": np.float32, "F16": np.float16, "BF16": np.uint16,
    "I64": np.int64, "I32": np.int32, "I16": np.int16, "I8": np.int8,
    "U64": np.uint64, "U32": np.uint32, "U16": np.uint16, "U8": np.uint8, "BOOL": np.bool_,
    "F8_E4M3": np.uint8, "F8_E5M2": np.uint8,
}
_TORCH2ST = {
    torch.float64: "F64", torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16",
    torch.int64: "I64", torch.int32: "I32", torch.int16: "I16", torch.int8: "I8",
    torch.uint8: "U8", torch.bool: "BOOL",
}
if hasattr(torch, "float8_e4m3fn"):
    _TORCH2ST[torch.float8_e4m3fn] = "F8_E4M3"
    _TORCH2ST[torch.float8_e5m2] = "F8_E5M2"


def read_header(path: str) -> Tuple[Dict[str, dict], int]:
    """Return (header dict without ``__metadata__`` removed, data start offset)."""
    with open(path, "rb") as f:
        raw = f.read(8)
        if len(raw) != 8:
            raise ValueError(f"{path}: truncated safetensors file")
        (n,) = struct.unpack("<Q", raw)
        if n > 512 * 1024 * 1024:
            raise ValueError(f"{path}: implausible header length {n}")
        header = json.loads(f.read(n).decode("utf-8"))
    return header, 8 + n


class SafetensorsFile:
    """Memory-mapped view of one ``.safetensors`` file."""

    def __init__(self, path: str):
        self.path = path
        self.header, self.data_start = read_header(path)
        self.metadata = self.header.pop("__metadata__", {}) or {}
        self._fh = open(path, "rb")
        size = os.fstat(self._fh.fileno()).st_size
        self._mm = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ) if size else None

    def keys(self) -> Iterable[str]:
        return self.header.keys()

    def __contains__(self, name: str) -> bool:
        return name in self.header

    def info(self, name: str) -> dict:
        return self.header[name]

    def shape(self, name: str) -> Tuple[int, ...]:
        return tuple(self.header[name]["shape"])

    def dtype_str(self, name: str) -> str:
        return self.header[name]["dtype"]

    def get_numpy(self, name: str) -> np.ndarray:
        ent = self.header[name]
        b, e = ent["data_offsets"]
        npdt = _ST2NP[ent["dtype"]]
        buf = np.frombuffer(self._mm, dtype=np.uint8, count=e - b, offset=self.data_start + b)
        return buf.view(npdt).reshape(ent["shape"])

    def get_tensor(self, name: str, *, copy: bool = True) -> torch.Tensor:
        ent = self.header[name]
        arr = self.get_numpy(name)
        st = ent["dtype"]
        if st == "BF16":
            t = torch.from_numpy(arr.view(np.int16).copy() if copy else arr.view(np.int16)).view(torch.bfloat16)
        elif st == "U32":
            t = torch.from_numpy(arr.view(np.int32).copy() if copy else arr.view(np.int32))
        elif st == "U16":
            t = torch.from_numpy(arr.view(np.int16).copy() if copy else arr.view(np.int16))
        elif st == "U64":
            t = torch.from_numpy(arr.view(np.int64).copy() if copy else arr.view(np.int64))
        elif st == "F8_E4M3":
            t = torch.from_numpy(arr.copy()).view(torch.float8_e4m3fn)
        elif st == "F8_E5M2":
            t = torch.from_numpy(arr.copy()).view(torch.float8_e5m2)
        else:
            t = torch.from_numpy(arr.copy() if copy else arr)
        return t

    def close(self) -> None:
        if self._mm is not None:
            try:
                self._mm.close()
            except BufferError:
                pass  # numpy views still alive; the OS reclaims the map at exit
            self._mm = None
        self._fh.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def load_file(path: str) -> Dict[str, torch.Tensor]:
    with SafetensorsFile(path) as f:
        return {k: f.get_tensor(k) for k in f.keys()}


def iter_tensors(path: str) -> Iterator[Tuple[str, torch.Tensor]]:
    with SafetensorsFile(path) as f:
        for k in list(f.keys()):
            yield k, f.get_tensor(k)


def _np_bytes(t) -> Tuple[str, Tuple[int, ...], bytes]:
    if isinstance(t, np.ndarray):
        for st, npdt in (("U32", np.uint32), ("U16", np.uint16), ("U8", np.uint8), ("I32", np.int32),
                         ("I64", np.int64), ("I16", np.int16), ("I8", np.int8), ("F32", np.float32),
                         ("F16", np.float16), ("F64", np.float64), ("BOOL", np.bool_), ("U64", np.uint64)):
            if t.dtype == npdt:
                return st, tuple(t.shape), np.ascontiguousarray(t).tobytes()
        raise TypeError(f"unsupported numpy dtype {t.dtype}")
    t = t.detach().cpu().contiguous()
    st = _TORCH2ST[t.dtype]
    if t.dtype == torch.bfloat16:
        raw = t.view(torch.int16).numpy().tobytes()
    elif st in ("F8_E4M3", "F8_E5M2"):
        raw = t.view(torch.uint8).numpy().tobytes()
    else:
        raw = t.numpy().tobytes()
    return st, tuple(t.shape), raw


def save_file(tensors: Mapping[str, object], path: str, metadata: Optional[Mapping[str, str]] = None,
              *, dtype_overrides: Optional[Mapping[str, str]] = None) -> None:
    """Write tensors (torch or numpy).  ``dtype_overrides`` relabels a tensor's
    header dtype without changing bytes (e.g. an ``int32`` torch tensor holding
    packed nibbles is stored as ``U32`` exactly as the reference's writers do)."""
    header: Dict[str, dict] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    blobs = []
    off = 0
    for name in tensors:
        st, shape, raw = _np_bytes(tensors[name])
        if dtype_overrides and name in dtype_overrides:
            st = dtype_overrides[name]
        header[name] = {"dtype": st, "shape": list(shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    hb = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hb += b" " * ((8 - len(hb) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(hb)))
        f.write(hb)
        for b in blobs:
            f.write(b)
    os.replace(tmp, path)
