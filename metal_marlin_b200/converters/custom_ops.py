"""Quantized custom operators for ONNX graphs (domain ``com.metal_marlin``): the operator definitions, a rewriter that
turns the MatMul nodes of a float model into quantized ones, and a session that runs the rewritten model.

``MarlinQuantizedMatMul(A, B_packed [K/8, N] uint32, scales [K/group, N] fp16) -> Y``, ``MarlinQuantizedLinear(X, W_packed, scales,
bias) -> Y`` and ``MarlinFlashAttention(Q, K, V [B, H, S, D]) -> O`` (attributes ``scale``, ``causal``).  ``compute`` takes and returns
NumPy arrays and runs this package's kernels (on the GPU when there is one).  The session is this package's graph
executor with the three operators added, behind the ``run(output_names, input_feed)`` call of an inference session;
``onnxruntime`` itself is not needed.

Parity: reference ``converters/ort_marlin_provider.py`` (``MarlinQuantizedMatMulOp`` :127, ``MarlinQuantizedLinearOp`` :207,
``MarlinFlashAttentionOp`` :278, ``create_session`` :437, ``export_with_marlin_ops`` :492).
"""
from __future__ import annotations

from pathlib import Path
from typing import Any, Dict, List, Optional, Sequence, Tuple, Union

import numpy as np
import torch

from . import onnx as _onnx

DOMAIN = "com.metal_marlin"
OPSET_VERSION = 1


def _device() -> torch.device:
    return torch.device("cuda" if torch.cuda.is_available() else "cpu")


def _t(a, dtype=None) -> torch.Tensor:
    if isinstance(a, torch.Tensor):
        t = a
    else:
        a = np.asarray(a)
        t = torch.from_numpy(a.view(np.int32) if a.dtype == np.uint32 else a)
    t = t.to(_device())
    return t.to(dtype) if dtype is not None else t


def _np(t: torch.Tensor, like) -> np.ndarray:
    dt = like.dtype if isinstance(like, np.ndarray) and like.dtype.kind == "f" else np.float16
    return t.float().cpu().numpy().astype(dt)


def _qmatmul(a: torch.Tensor, packed: torch.Tensor, scales: torch.Tensor, group_size: int) -> torch.Tensor:
    from ..compat_api import marlin_gemm_fp4
    return marlin_gemm_fp4(a, packed, scales.to(torch.float16), group_size)


class MarlinQuantizedMatMulOp:
    op_type, domain = "MarlinQuantizedMatMul", DOMAIN

    @staticmethod
    def get_inputs() -> List[Tuple[str, str]]:
        return [("A", "tensor(float16)"), ("B_packed", "tensor(uint32)"), ("scales", "tensor(float16)")]

    @staticmethod
    def get_outputs() -> List[Tuple[str, str]]:
        return [("Y", "tensor(float16)")]

    @staticmethod
    def get_attrs() -> Dict[str, Tuple[str, Any]]:
        return {"group_size": ("int", 128)}

    @staticmethod
    def compute(A, B_packed, scales, *, group_size: int = 128):
        return _np(_qmatmul(_t(A), _t(B_packed), _t(scales), group_size), A)


class MarlinQuantizedLinearOp:
    op_type, domain = "MarlinQuantizedLinear", DOMAIN

    @staticmethod
    def get_inputs() -> List[Tuple[str, str]]:
        return [("X", "tensor(float16)"), ("W_packed", "tensor(uint32)"), ("scales", "tensor(float16)"), ("bias", "tensor(float16)")]

    @staticmethod
    def get_outputs() -> List[Tuple[str, str]]:
        return [("Y", "tensor(float16)")]

    @staticmethod
    def get_attrs() -> Dict[str, Tuple[str, Any]]:
        return {"group_size": ("int", 128)}

    @staticmethod
    def compute(X, W_packed, scales, bias=None, *, group_size: int = 128):
        y = _qmatmul(_t(X), _t(W_packed), _t(scales), group_size)
        if bias is not None and np.size(bias):
            y = y + _t(bias, y.dtype)
        return _np(y, X)


class MarlinFlashAttentionOp:
    op_type, domain = "MarlinFlashAttention", DOMAIN

    @staticmethod
    def get_inputs() -> List[Tuple[str, str]]:
        return [("Q", "tensor(float16)"), ("K", "tensor(float16)"), ("V", "tensor(float16)")]

    @staticmethod
    def get_outputs() -> List[Tuple[str, str]]:
        return [("O", "tensor(float16)")]

    @staticmethod
    def get_attrs() -> Dict[str, Tuple[str, Any]]:
        return {"scale": ("float", 0.0), "causal": ("int", 0)}

    @staticmethod
    def compute(Q, K, V, *, scale: float = 0.0, causal: int = 0):
        from ..compat_api import flash_attention_metal
        q, k, v = (_t(x, torch.bfloat16 if _device().type == "cuda" else torch.float32) for x in (Q, K, V))
        return _np(flash_attention_metal(q, k, v, scale=scale or None, causal=bool(causal)), Q)


CUSTOM_OPS = {c.op_type: c for c in (MarlinQuantizedMatMulOp, MarlinQuantizedLinearOp, MarlinFlashAttentionOp)}


def export_with_marlin_ops(onnx_model_path: Union[str, Path, bytes], output_path: Optional[Union[str, Path]],
                           weights: Optional[Dict[str, Tuple[np.ndarray, np.ndarray]]] = None, *, group_size: int = 128) -> bytes:
    """Rewrite a float ONNX model: every ``MatMul`` whose second input is an initializer named in ``weights`` (``{name: (packed
    uint32 [K/8, N], scales fp16 [K/group, N])}``) becomes a ``MarlinQuantizedMatMul``; a following ``Add`` with a constant bias is
    folded into ``MarlinQuantizedLinear``.  ``weights=None`` packs every eligible 2-D MatMul initializer here.  The float
    initializer is dropped once nothing else reads it.  Returns the serialized model (also written to ``output_path``)."""
    from ..compat_api import pack_fp4_weights
    g = _onnx.load_onnx(onnx_model_path)
    if weights is None:
        weights = {}
        for n in g.nodes:
            w = g.initializers.get(n.inputs[1]) if n.op_type == "MatMul" and len(n.inputs) > 1 else None
            if w is not None and w.ndim == 2 and w.shape[0] % group_size == 0 and w.shape[1] % 16 == 0:
                packed, scales, _meta = pack_fp4_weights(np.asarray(w, dtype=np.float32), group_size)
                weights[n.inputs[1]] = (packed, scales)
    readers: Dict[str, int] = {}
    for n in g.nodes:
        for i in n.inputs:
            readers[i] = readers.get(i, 0) + 1
    nodes: List[_onnx.ONNXOp] = []
    skip = set()
    for idx, n in enumerate(g.nodes):
        if idx in skip:
            continue
        if n.op_type != "MatMul" or len(n.inputs) < 2 or n.inputs[1] not in weights:
            nodes.append(n)
            continue
        wname = n.inputs[1]
        packed, scales = weights[wname]
        g.initializers[wname + "_packed"] = np.ascontiguousarray(np.asarray(packed)).view(np.uint32)
        g.initializers[wname + "_scales"] = np.asarray(scales, dtype=np.float16)
        readers[wname] -= 1
        nxt = g.nodes[idx + 1] if idx + 1 < len(g.nodes) else None
        bias = None
        if nxt is not None and nxt.op_type == "Add" and readers.get(n.outputs[0], 0) == 1 and n.outputs[0] in nxt.inputs:
            other = [i for i in nxt.inputs if i != n.outputs[0]]
            if len(other) == 1 and other[0] in g.initializers and g.initializers[other[0]].ndim == 1:
                bias = other[0]
        if bias is not None:
            nodes.append(_onnx.ONNXOp(n.name, "MarlinQuantizedLinear", [n.inputs[0], wname + "_packed", wname + "_scales", bias], list(nxt.outputs),
                                      {"group_size": int(group_size)}, DOMAIN))
            skip.add(idx + 1)
        else:
            nodes.append(_onnx.ONNXOp(n.name, "MarlinQuantizedMatMul", [n.inputs[0], wname + "_packed", wname + "_scales"], list(n.outputs),
                                      {"group_size": int(group_size)}, DOMAIN))
    for wname in weights:
        if readers.get(wname, 0) <= 0:
            g.initializers.pop(wname, None)
    g.nodes = nodes
    return _onnx.save_onnx(g, output_path)


class _Executor(_onnx.ONNXExecutor):
    """The graph executor with the custom-domain operators; packed weights are turned into device weights once."""

    def __init__(self, graph: _onnx.ONNXGraph, device=None):
        super().__init__(graph, quantize=None, device=device or _device(), dtype=torch.float32)
        self._weights: Dict[str, Any] = {}
        self._table.update({"MarlinQuantizedMatMul": self._q_matmul, "MarlinQuantizedLinear": self._q_linear, "MarlinFlashAttention": self._attention})

    def _weight(self, packed_name: str, scales_name: str):
        W = self._weights.get(packed_name)
        if W is None:
            from ..ops.weights import FP4Weight
            packed = torch.from_numpy(np.asarray(self.graph.initializers[packed_name]).view(np.int32))
            scales = torch.from_numpy(np.asarray(self.graph.initializers[scales_name], dtype=np.float16))
            W = self._weights[packed_name] = FP4Weight.from_marlin_fp4(packed, scales, self.device)
        return W

    def _mm(self, n, x):
        from .. import ops
        W = self._weight(n.inputs[1], n.inputs[2])
        y = ops.linear(x.reshape(-1, x.shape[-1]).to(torch.bfloat16), W)
        return y.to(x.dtype).reshape(*x.shape[:-1], -1)

    def _q_matmul(self, n, a):
        return [self._mm(n, a[0])]

    def _q_linear(self, n, a):
        y = self._mm(n, a[0])
        return [y + a[3].to(y.dtype) if len(a) > 3 and a[3] is not None else y]

    def _attention(self, n, a):
        from ..compat_api import flash_attention_metal
        dt = torch.bfloat16 if self.device.type == "cuda" else torch.float32
        o = flash_attention_metal(a[0].to(dt), a[1].to(dt), a[2].to(dt), scale=float(n.attrs.get("scale", 0.0)) or None,
                                  causal=bool(int(n.attrs.get("causal", 0))))
        return [o.to(a[0].dtype)]


class MarlinSession:
    """``run(output_names, input_feed)`` / ``get_inputs()`` / ``get_outputs()`` over the executor (NumPy in, NumPy out)."""

    class _Arg:
        def __init__(self, name: str):
            self.name = name

    def __init__(self, model: Union[str, Path, bytes], device=None):
        self.graph = _onnx.load_onnx(model)
        self.executor = _Executor(self.graph, device)

    def get_inputs(self):
        return [self._Arg(n) for n in self.graph.inputs]

    def get_outputs(self):
        return [self._Arg(n) for n in self.graph.outputs]

    def run(self, output_names: Optional[Sequence[str]], input_feed: Dict[str, np.ndarray]) -> List[np.ndarray]:
        feed = {}
        for k, v in input_feed.items():
            t = torch.from_numpy(np.asarray(v))
            feed[k] = t.float() if t.is_floating_point() else t
        with torch.no_grad():
            out = self.executor(**feed)
        like = next(iter(input_feed.values()))
        names = list(output_names) if output_names else self.graph.outputs
        res = []
        for n in names:
            t = out[n]
            res.append(_np(t, np.asarray(like)) if t.is_floating_point() else t.cpu().numpy())
        return res


def create_session(model_path: Union[str, Path, bytes], *, group_size: int = 128, use_extensions: bool = True,
                   custom_lib_path: Optional[Union[str, Path]] = None, device=None) -> MarlinSession:
    """A session for a model that uses the ``com.metal_marlin`` operators.  ``group_size`` is read from each node's attribute;
    ``use_extensions`` / ``custom_lib_path`` (a compiled operator library for another runtime) are accepted for signature
    compatibility — a path that does not exist is still an error."""
    if custom_lib_path is not None and not Path(custom_lib_path).exists():
        raise FileNotFoundError(f"custom operator library not found: {custom_lib_path}")
    return MarlinSession(model_path, device)
