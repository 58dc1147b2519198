"""ONNX import without the ``onnx`` package: a protobuf wire-format reader (and a small writer, used by the tests and by
``export_linear_stack``) for the subset of ``onnx.proto`` a weight importer needs, a graph summary with architecture
detection, and an executor that runs the graph with PyTorch ops while MatMul / Gemm nodes whose weight is an initializer
go through this package's quantized linears (FP4 tile layout on the GPU, RTN-quantized on load).

Parity: reference ``metal_marlin/onnx_graph.py:25-561`` (``ONNXOp``, ``parse_onnx_graph``, ``detect_architecture``,
``summarize_graph``), ``metal_marlin/onnx_loader.py`` (initializer extraction) and
``metal_marlin/converters/onnx_executor.py:88-632`` (``ONNXGraph``, ``ONNXExecutor.from_file`` / ``__call__``, node handlers).
The ONNX-Runtime execution-provider shim of the reference (``converters/ort_marlin_provider.py``) has no counterpart:
ONNX Runtime is not a dependency here, the executor below is the way to run an imported graph.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Dict, List, Optional, Sequence, Tuple, Union

import numpy as np
import torch
import torch.nn.functional as F

# ---------------------------------------------------------------------------------------------------------------
# protobuf wire format
# ---------------------------------------------------------------------------------------------------------------
_VARINT, _I64, _LEN, _I32 = 0, 1, 2, 5


def _read_varint(buf: memoryview, pos: int) -> Tuple[int, int]:
    out = shift = 0
    while True:
        b = buf[pos]
        pos += 1
        out |= (b & 0x7F) << shift
        if not b & 0x80:
            return out, pos
        shift += 7


def _fields(buf: memoryview):
    """Yields ``(field number, wire type, value)``; length-delimited values are memoryviews."""
    pos, n = 0, len(buf)
    while pos < n:
        key, pos = _read_varint(buf, pos)
        fno, wt = key >> 3, key & 7
        if wt == _VARINT:
            v, pos = _read_varint(buf, pos)
        elif wt == _I64:
            v, pos = bytes(buf[pos:pos + 8]), pos + 8
        elif wt == _LEN:
            ln, pos = _read_varint(buf, pos)
            v, pos = buf[pos:pos + ln], pos + ln
        elif wt == _I32:
            v, pos = bytes(buf[pos:pos + 4]), pos + 4
        else:
            raise ValueError(f"unsupported protobuf wire type {wt}")
        yield fno, wt, v


def _signed(v: int) -> int:
    return v - (1 << 64) if v >= (1 << 63) else v


def _packed_varints(v) -> List[int]:
    out, pos, n = [], 0, len(v)
    while pos < n:
        x, pos = _read_varint(v, pos)
        out.append(_signed(x))
    return out


def _w_varint(x: int) -> bytes:
    x &= (1 << 64) - 1
    out = bytearray()
    while True:
        b = x & 0x7F
        x >>= 7
        if x:
            out.append(b | 0x80)
        else:
            out.append(b)
            return bytes(out)


def _w_field(fno: int, wt: int, payload: Union[int, bytes]) -> bytes:
    key = _w_varint((fno << 3) | wt)
    if wt == _VARINT:
        return key + _w_varint(int(payload))
    if wt == _LEN:
        return key + _w_varint(len(payload)) + bytes(payload)
    return key + bytes(payload)


# ONNX TensorProto.DataType -> numpy
_DTYPES = {1: np.float32, 2: np.uint8, 3: np.int8, 5: np.int16, 6: np.int32, 7: np.int64, 9: np.bool_, 10: np.float16,
           11: np.float64, 12: np.uint32, 13: np.uint64}
_DTYPE_CODE = {np.dtype(v): k for k, v in _DTYPES.items()}
_BF16 = 16


def _parse_tensor(buf: memoryview) -> Tuple[str, np.ndarray]:
    dims: List[int] = []
    dtype, name, raw = 1, "", None
    floats: List[float] = []
    ints: List[int] = []
    for fno, wt, v in _fields(buf):
        if fno == 1:
            dims += _packed_varints(v) if wt == _LEN else [_signed(v)]
        elif fno == 2:
            dtype = v
        elif fno == 4:        # float_data
            floats += list(np.frombuffer(bytes(v), dtype="<f4")) if wt == _LEN else [struct.unpack("<f", v)[0]]
        elif fno in (5, 7):   # int32_data / int64_data
            ints += _packed_varints(v) if wt == _LEN else [_signed(v)]
        elif fno == 8:
            name = bytes(v).decode()
        elif fno == 9:
            raw = bytes(v)
    if dtype == _BF16:
        src = np.frombuffer(raw, dtype="<u2") if raw is not None else np.asarray(ints, dtype=np.uint16)
        arr = (src.astype(np.uint32) << 16).view(np.float32)
    else:
        np_dt = _DTYPES.get(dtype)
        if np_dt is None:
            raise ValueError(f"unsupported ONNX tensor data type {dtype}")
        if raw is not None:
            arr = np.frombuffer(raw, dtype=np.dtype(np_dt).newbyteorder("<"))
        elif floats:
            arr = np.asarray(floats, dtype=np_dt)
        else:
            arr = np.asarray(ints, dtype=np_dt)
    return name, arr.reshape(dims if dims else ()).copy()


def _parse_attribute(buf: memoryview) -> Tuple[str, Any]:
    name, val = "", None
    floats: List[float] = []
    ints: List[int] = []
    strs: List[str] = []
    for fno, wt, v in _fields(buf):
        if fno == 1:
            name = bytes(v).decode()
        elif fno == 2:
            val = struct.unpack("<f", v)[0]
        elif fno == 3:
            val = _signed(v)
        elif fno == 4:
            val = bytes(v).decode(errors="replace")
        elif fno == 5:
            val = _parse_tensor(v)[1]
        elif fno == 7:
            floats += list(np.frombuffer(bytes(v), dtype="<f4")) if wt == _LEN else [struct.unpack("<f", v)[0]]
        elif fno == 8:
            ints += _packed_varints(v) if wt == _LEN else [_signed(v)]
        elif fno == 9:
            strs.append(bytes(v).decode(errors="replace"))
    if val is None:
        val = ints if ints else (floats if floats else (strs if strs else None))
    return name, val


@dataclass
class ONNXOp:
    """One node of the graph (reference ``onnx_graph.py:25``)."""
    name: str
    op_type: str
    inputs: List[str]
    outputs: List[str]
    attrs: Dict[str, Any] = field(default_factory=dict)
    domain: str = ""               # operator set the node belongs to ("" = the standard ONNX set)


ONNXNode = ONNXOp


@dataclass
class ONNXGraph:
    nodes: List[ONNXOp]
    initializers: Dict[str, np.ndarray]
    inputs: List[str]
    outputs: List[str]
    name: str = ""
    opset: int = 0


def _parse_node(buf: memoryview) -> ONNXOp:
    ins, outs, attrs, name, op, domain = [], [], {}, "", "", ""
    for fno, _, v in _fields(buf):
        if fno == 1:
            ins.append(bytes(v).decode())
        elif fno == 2:
            outs.append(bytes(v).decode())
        elif fno == 3:
            name = bytes(v).decode()
        elif fno == 4:
            op = bytes(v).decode()
        elif fno == 5:
            k, a = _parse_attribute(v)
            attrs[k] = a
        elif fno == 7:
            domain = bytes(v).decode()
    return ONNXOp(name or (outs[0] if outs else op), op, ins, outs, attrs, domain)


def _value_info_name(buf: memoryview) -> str:
    for fno, _, v in _fields(buf):
        if fno == 1:
            return bytes(v).decode()
    return ""


def load_onnx(path_or_bytes: Union[str, Path, bytes]) -> ONNXGraph:
    """Parse a ``ModelProto`` (file path or bytes)."""
    data = Path(path_or_bytes).read_bytes() if not isinstance(path_or_bytes, (bytes, bytearray)) else bytes(path_or_bytes)
    graph_buf, opset = None, 0
    for fno, _, v in _fields(memoryview(data)):
        if fno == 7:
            graph_buf = v
        elif fno == 8:        # opset_import: OperatorSetIdProto {domain = 1, version = 2}; custom domains carry their own versions
            dom, ver = "", 0
            for f2, _, v2 in _fields(v):
                if f2 == 1:
                    dom = bytes(v2).decode()
                elif f2 == 2:
                    ver = int(v2)
            if dom in ("", "ai.onnx"):
                opset = max(opset, ver)
    if graph_buf is None:
        raise ValueError("not an ONNX ModelProto: no graph")
    nodes, inits, ins, outs, gname = [], {}, [], [], ""
    for fno, _, v in _fields(graph_buf):
        if fno == 1:
            nodes.append(_parse_node(v))
        elif fno == 2:
            gname = bytes(v).decode()
        elif fno == 5:
            k, arr = _parse_tensor(v)
            inits[k] = arr
        elif fno == 11:
            ins.append(_value_info_name(v))
        elif fno == 12:
            outs.append(_value_info_name(v))
    return ONNXGraph(nodes, inits, [i for i in ins if i not in inits], outs, gname, opset)


def parse_onnx_graph(path_or_bytes) -> List[ONNXOp]:
    return load_onnx(path_or_bytes).nodes


# ---------------------------------------------------------------------------------------------------------------
# writer (tests, small exports)
# ---------------------------------------------------------------------------------------------------------------
def _tensor_proto(name: str, arr: np.ndarray) -> bytes:
    arr = np.asarray(arr, order="C")      # (ascontiguousarray would turn a scalar into a 1-element vector)
    out = b"".join(_w_field(1, _VARINT, d) for d in arr.shape)
    out += _w_field(2, _VARINT, _DTYPE_CODE[arr.dtype]) + _w_field(8, _LEN, name.encode()) + _w_field(9, _LEN, arr.tobytes())
    return out


def _attr_proto(name: str, val: Any) -> bytes:
    out = _w_field(1, _LEN, name.encode())
    if isinstance(val, float):
        return out + _w_field(2, _I32, struct.pack("<f", val)) + _w_field(20, _VARINT, 1)
    if isinstance(val, int):
        return out + _w_field(3, _VARINT, val) + _w_field(20, _VARINT, 2)
    if isinstance(val, str):
        return out + _w_field(4, _LEN, val.encode()) + _w_field(20, _VARINT, 3)
    if isinstance(val, np.ndarray):
        return out + _w_field(5, _LEN, _tensor_proto("", val)) + _w_field(20, _VARINT, 4)
    if isinstance(val, (list, tuple)) and all(isinstance(x, int) for x in val):
        return out + b"".join(_w_field(8, _VARINT, x) for x in val) + _w_field(20, _VARINT, 7)
    if isinstance(val, (list, tuple)):
        return out + b"".join(_w_field(7, _I32, struct.pack("<f", float(x))) for x in val) + _w_field(20, _VARINT, 6)
    raise TypeError(type(val))


def save_onnx(graph: ONNXGraph, path: Optional[Union[str, Path]] = None) -> bytes:
    """Serialize (enough of) a ModelProto for :func:`load_onnx` and for other ONNX readers."""
    g = b""
    for n in graph.nodes:
        nb = b"".join(_w_field(1, _LEN, i.encode()) for i in n.inputs) + b"".join(_w_field(2, _LEN, o.encode()) for o in n.outputs)
        nb += _w_field(3, _LEN, n.name.encode()) + _w_field(4, _LEN, n.op_type.encode())
        nb += b"".join(_w_field(5, _LEN, _attr_proto(k, v)) for k, v in n.attrs.items())
        if n.domain:
            nb += _w_field(7, _LEN, n.domain.encode())
        g += _w_field(1, _LEN, nb)
    g += _w_field(2, _LEN, (graph.name or "graph").encode())
    for k, arr in graph.initializers.items():
        g += _w_field(5, _LEN, _tensor_proto(k, arr))
    for i in graph.inputs:
        g += _w_field(11, _LEN, _w_field(1, _LEN, i.encode()))
    for o in graph.outputs:
        g += _w_field(12, _LEN, _w_field(1, _LEN, o.encode()))
    model = _w_field(1, _VARINT, 8) + _w_field(7, _LEN, g) + _w_field(8, _LEN, _w_field(2, _VARINT, graph.opset or 17))
    for dom in sorted({n.domain for n in graph.nodes if n.domain}):
        model += _w_field(8, _LEN, _w_field(1, _LEN, dom.encode()) + _w_field(2, _VARINT, 1))
    if path is not None:
        Path(path).write_bytes(model)
    return model


# ---------------------------------------------------------------------------------------------------------------
# graph analysis
# ---------------------------------------------------------------------------------------------------------------
def _count_op_types(ops: Sequence[ONNXOp]) -> Dict[str, int]:
    out: Dict[str, int] = {}
    for o in ops:
        out[o.op_type] = out.get(o.op_type, 0) + 1
    return out


def detect_architecture(ops: Sequence[ONNXOp]) -> str:
    """Coarse family from the op mix: ``moe`` (TopK / routing gathers beside MatMuls), ``llama`` (RMS-norm pattern:
    Pow + ReduceMean + Sqrt/Rsqrt without LayerNormalization, SiLU gating), ``bert`` (LayerNormalization + Erf/Gelu, no
    causal Trilu), ``gpt`` (LayerNormalization + causal masking), ``transformer`` (attention-like Softmax between
    MatMuls), else ``unknown``."""
    c = _count_op_types(ops)
    has = lambda *names: any(n in c for n in names)
    if not has("MatMul", "Gemm", "MatMulNBits"):
        return "unknown"
    if has("TopK") and has("Softmax", "Sigmoid") and has("Gather", "GatherElements", "ScatterND", "ScatterElements"):
        return "moe"
    rms = (has("Pow") and has("ReduceMean") and has("Sqrt", "Reciprocal", "Rsqrt")) or has("SimplifiedLayerNormalization", "RMSNormalization")
    if rms and not has("LayerNormalization") and (has("Sigmoid", "Silu") or has("RotaryEmbedding")):
        return "llama"
    if has("LayerNormalization") or (has("ReduceMean") and has("Sub") and has("Sqrt")):
        if has("Trilu", "Where") and not has("Erf"):
            return "gpt"
        if has("Erf", "Gelu", "Tanh"):
            return "bert" if not has("Trilu") else "gpt"
    if has("Softmax") and c.get("MatMul", 0) + c.get("Gemm", 0) >= 4:
        return "transformer"
    return "unknown"


def get_layer_count(ops: Sequence[ONNXOp]) -> int:
    """Attention blocks = Softmax nodes that sit between two MatMuls (one per layer in a decoder / encoder stack)."""
    return max(sum(1 for o in ops if o.op_type in ("Softmax", "Attention", "MultiHeadAttention", "GroupQueryAttention")), 0)


def summarize_graph(ops: Sequence[ONNXOp]) -> Dict[str, Any]:
    c = _count_op_types(ops)
    return {"num_ops": len(ops), "op_counts": dict(sorted(c.items(), key=lambda kv: -kv[1])), "architecture": detect_architecture(ops),
            "layers": get_layer_count(ops), "matmuls": c.get("MatMul", 0) + c.get("Gemm", 0)}


def extract_linear_weights(graph: ONNXGraph, min_features: int = 16) -> Dict[str, torch.Tensor]:
    """``{initializer name: weight [out, in]}`` of every MatMul / Gemm whose second operand is a 2-D initializer (the
    tensors a weight-only quantizer converts; reference ``onnx_loader.py``)."""
    out: Dict[str, torch.Tensor] = {}
    for n in graph.nodes:
        if n.op_type not in ("MatMul", "Gemm") or len(n.inputs) < 2 or n.inputs[1] not in graph.initializers:
            continue
        w = graph.initializers[n.inputs[1]]
        if w.ndim != 2 or min(w.shape) < min_features:
            continue
        wt = torch.from_numpy(np.asarray(w, dtype=np.float32))
        trans_b = n.op_type == "Gemm" and int(n.attrs.get("transB", 0)) == 1
        out[n.inputs[1]] = wt if trans_b else wt.t().contiguous()        # MatMul computes x @ W with W [in, out]
    return out


# ---------------------------------------------------------------------------------------------------------------
# executor
# ---------------------------------------------------------------------------------------------------------------
class ONNXExecutor:
    """Runs the graph node by node.  ``quantize="fp4"`` converts every eligible MatMul / Gemm weight (both dims multiples
    of ``group_size`` / 16) to this package's FP4 linear; other nodes are PyTorch ops."""

    def __init__(self, graph: ONNXGraph, quantize: Optional[str] = "fp4", group_size: int = 128, device: Union[str, torch.device] = "cpu",
                 dtype: torch.dtype = torch.float32):
        self.graph, self.device, self.dtype = graph, torch.device(device), dtype
        self.consts: Dict[str, torch.Tensor] = {}
        self.linears: Dict[str, Any] = {}
        lin = extract_linear_weights(graph) if quantize else {}
        for k, arr in graph.initializers.items():
            t = torch.from_numpy(np.asarray(arr))
            self.consts[k] = t.to(self.device, dtype if t.is_floating_point() else t.dtype)
        if quantize:
            from ..layers import MMFP4Linear
            for k, w in lin.items():
                out_f, in_f = w.shape
                if quantize == "fp4" and in_f % 64 == 0 and out_f % 16 == 0:
                    gs = group_size if in_f % group_size == 0 else 64
                    self.linears[k] = MMFP4Linear.from_float(w, group_size=gs, device=self.device)
        self._table = self._build_dispatch_table()

    @classmethod
    def from_file(cls, path, quantize: Optional[str] = "fp4", **kw) -> "ONNXExecutor":
        return cls(load_onnx(path), quantize=quantize, **kw)

    # ------------------------------------------------------------------ running
    def __call__(self, **inputs: torch.Tensor) -> Dict[str, torch.Tensor]:
        vals: Dict[str, torch.Tensor] = dict(self.consts)
        for k, v in inputs.items():
            vals[k] = v.to(self.device)
        missing = [i for i in self.graph.inputs if i not in vals]
        if missing:
            raise KeyError(f"missing graph inputs: {missing}")
        for n in self.graph.nodes:
            fn = self._table.get(n.op_type)
            if fn is None:
                raise NotImplementedError(f"ONNX op {n.op_type} (node {n.name})")
            args = [vals[i] if i else None for i in n.inputs]
            res = fn(n, args)
            for o, r in zip(n.outputs, res):
                if o:
                    vals[o] = r
        return {o: vals[o] for o in self.graph.outputs}

    def _linear(self, key: str, x: torch.Tensor) -> torch.Tensor:
        lin = self.linears[key]
        shp = x.shape
        y = lin(x.reshape(-1, shp[-1]).to(torch.bfloat16 if self.device.type == "cuda" else x.dtype))
        return y.to(x.dtype).reshape(*shp[:-1], y.shape[-1])

    def _matmul(self, n: ONNXOp, a):
        if n.inputs[1] in self.linears:
            return [self._linear(n.inputs[1], a[0])]
        return [torch.matmul(a[0], a[1])]

    def _gemm(self, n: ONNXOp, a):
        alpha, beta = float(n.attrs.get("alpha", 1.0)), float(n.attrs.get("beta", 1.0))
        x = a[0].t() if int(n.attrs.get("transA", 0)) else a[0]
        if n.inputs[1] in self.linears and alpha == 1.0:
            y = self._linear(n.inputs[1], x)
        else:
            w = a[1].t() if int(n.attrs.get("transB", 0)) else a[1]
            y = alpha * (x @ w)
        if len(a) > 2 and a[2] is not None:
            y = y + beta * a[2]
        return [y]

    def _build_dispatch_table(self) -> Dict[str, Any]:
        def axes_of(n, a, idx=1):
            if "axes" in n.attrs:
                return [int(x) for x in n.attrs["axes"]]
            if len(a) > idx and a[idx] is not None:
                return [int(x) for x in a[idx].reshape(-1).tolist()]
            return None

        def reduce(fn):
            def run(n, a):
                ax = axes_of(n, a)
                keep = bool(int(n.attrs.get("keepdims", 1)))
                return [fn(a[0], dim=ax, keepdim=keep) if ax is not None else fn(a[0]).reshape([1] * a[0].dim() if keep else [])]
            return run

        def layernorm(n, a):
            axis = int(n.attrs.get("axis", -1))
            dims = list(range(axis % a[0].dim(), a[0].dim()))
            shape = [a[0].shape[d] for d in dims]
            return [F.layer_norm(a[0], shape, a[1], a[2] if len(a) > 2 else None, float(n.attrs.get("epsilon", 1e-5)))]

        def rmsnorm(n, a):
            eps = float(n.attrs.get("epsilon", 1e-6))
            x = a[0].float()
            return [(x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * a[1].float()).to(a[0].dtype)]

        def split(n, a):
            axis = int(n.attrs.get("axis", 0))
            if len(a) > 1 and a[1] is not None:
                sizes = [int(x) for x in a[1].tolist()]
            elif "split" in n.attrs:
                sizes = [int(x) for x in n.attrs["split"]]
            else:
                k = len(n.outputs)
                sizes = [a[0].shape[axis] // k] * k
            return list(torch.split(a[0], sizes, dim=axis))

        def squeeze(n, a):
            ax = axes_of(n, a)
            x = a[0]
            if ax is None:
                return [x.squeeze()]
            for d in sorted([d % x.dim() for d in ax], reverse=True):
                x = x.squeeze(d)
            return [x]

        def unsqueeze(n, a):
            x = a[0]
            for d in sorted(axes_of(n, a)):
                x = x.unsqueeze(d)
            return [x]

        def cast(n, a):
            to = int(n.attrs.get("to", 1))
            tdt = {1: torch.float32, 6: torch.int32, 7: torch.int64, 9: torch.bool, 10: torch.float16, 11: torch.float64, 16: torch.bfloat16}[to]
            return [a[0].to(tdt)]

        def constant(n, a):
            v = n.attrs.get("value")
            if v is None:
                v = np.asarray(n.attrs.get("value_float", n.attrs.get("value_int", n.attrs.get("value_ints", n.attrs.get("value_floats")))))
            t = torch.from_numpy(np.asarray(v))
            return [t.to(self.device, self.dtype if t.is_floating_point() else t.dtype)]

        def gelu(n, a):
            return [F.gelu(a[0], approximate="tanh" if n.attrs.get("approximate") == "tanh" else "none")]

        def slice_(n, a):
            starts, ends = a[1].tolist(), a[2].tolist()
            axes = a[3].tolist() if len(a) > 3 and a[3] is not None else list(range(len(starts)))
            steps = a[4].tolist() if len(a) > 4 and a[4] is not None else [1] * len(starts)
            x = a[0]
            for s, e, ax, st in zip(starts, ends, axes, steps):
                idx = [slice(None)] * x.dim()
                idx[ax] = slice(int(s), int(min(e, x.shape[ax])) if e >= 0 else int(e), int(st))
                x = x[tuple(idx)]
            return [x]

        un = lambda f: (lambda n, a: [f(a[0])])
        bi = lambda f: (lambda n, a: [f(a[0], a[1])])
        return {
            "MatMul": self._matmul, "Gemm": self._gemm, "Add": bi(torch.add), "Sub": bi(torch.sub), "Mul": bi(torch.mul), "Div": bi(torch.div),
            "Pow": bi(torch.pow), "Sqrt": un(torch.sqrt), "Reciprocal": un(torch.reciprocal), "Neg": un(torch.neg), "Exp": un(torch.exp),
            "Erf": un(torch.erf), "Relu": un(F.relu), "Sigmoid": un(torch.sigmoid), "Tanh": un(torch.tanh), "Gelu": gelu,
            "Silu": un(F.silu), "Identity": un(lambda x: x), "Softmax": lambda n, a: [torch.softmax(a[0], int(n.attrs.get("axis", -1)))],
            "LayerNormalization": layernorm, "SimplifiedLayerNormalization": rmsnorm, "RMSNormalization": rmsnorm,
            "Reshape": lambda n, a: [a[0].reshape([int(s) if s != 0 else a[0].shape[i] for i, s in enumerate(a[1].tolist())])],
            "Transpose": lambda n, a: [a[0].permute(*[int(p) for p in n.attrs.get("perm", list(range(a[0].dim()))[::-1])])],
            "Concat": lambda n, a: [torch.cat(a, dim=int(n.attrs.get("axis", 0)))], "Split": split, "Squeeze": squeeze, "Unsqueeze": unsqueeze,
            "Gather": lambda n, a: [torch.index_select(a[0], int(n.attrs.get("axis", 0)), a[1].reshape(-1).long()).reshape(
                *a[0].shape[:int(n.attrs.get("axis", 0)) % a[0].dim()], *a[1].shape, *a[0].shape[int(n.attrs.get("axis", 0)) % a[0].dim() + 1:])],
            "ReduceMean": reduce(torch.mean), "ReduceSum": reduce(torch.sum), "Cast": cast, "Constant": constant, "Slice": slice_,
            "Where": lambda n, a: [torch.where(a[0].bool(), a[1], a[2])], "Shape": lambda n, a: [torch.tensor(list(a[0].shape), dtype=torch.int64,
                                                                                                           device=self.device)],
        }


def export_linear_stack(weights: Sequence[torch.Tensor], biases: Optional[Sequence[Optional[torch.Tensor]]] = None, activation: str = "Relu",
                        path: Optional[Union[str, Path]] = None) -> bytes:
    """ONNX model of an MLP ``x -> act(x W0^T + b0) -> ...`` (weights ``[out, in]``): a small producer for round-trip tests
    and for handing converted stacks to other runtimes."""
    nodes, inits, cur = [], {}, "x"
    for i, w in enumerate(weights):
        inits[f"w{i}"] = w.t().contiguous().float().numpy()
        nodes.append(ONNXOp(f"mm{i}", "MatMul", [cur, f"w{i}"], [f"h{i}"]))
        cur = f"h{i}"
        if biases is not None and biases[i] is not None:
            inits[f"b{i}"] = biases[i].float().numpy()
            nodes.append(ONNXOp(f"add{i}", "Add", [cur, f"b{i}"], [f"hb{i}"]))
            cur = f"hb{i}"
        if i + 1 < len(weights):
            nodes.append(ONNXOp(f"act{i}", activation, [cur], [f"a{i}"]))
            cur = f"a{i}"
    return save_onnx(ONNXGraph(nodes, inits, ["x"], [cur], "linear_stack", 17), path)
