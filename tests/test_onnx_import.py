"""ONNX import: wire-format round trip, attributes, graph summary, executor against plain PyTorch (reference:
tests/test_onnx_graph.py, tests/test_onnx_executor.py with its tiny fixture models)."""
import numpy as np
import torch

from metal_marlin_b200.converters import onnx as ox


def _attention_block_graph(hidden=64, heads=4):
    rng = np.random.default_rng(0)
    w = lambda *s: (rng.standard_normal(s) * 0.1).astype(np.float32)
    inits = {"wq": w(hidden, hidden), "wk": w(hidden, hidden), "wv": w(hidden, hidden), "wo": w(hidden, hidden),
             "ln_g": np.ones(hidden, np.float32), "ln_b": np.zeros(hidden, np.float32),
             "shape_h": np.array([0, 0, heads, hidden // heads], np.int64), "shape_m": np.array([0, 0, hidden], np.int64),
             "scale": np.array(1.0 / np.sqrt(hidden // heads), np.float32)}
    N = ox.ONNXOp
    nodes = [
        N("ln", "LayerNormalization", ["x", "ln_g", "ln_b"], ["xn"], {"axis": -1, "epsilon": 1e-5}),
        N("q", "MatMul", ["xn", "wq"], ["q"]), N("k", "MatMul", ["xn", "wk"], ["k"]), N("v", "MatMul", ["xn", "wv"], ["v"]),
        N("qr", "Reshape", ["q", "shape_h"], ["q4"]), N("kr", "Reshape", ["k", "shape_h"], ["k4"]), N("vr", "Reshape", ["v", "shape_h"], ["v4"]),
        N("qt", "Transpose", ["q4"], ["qh"], {"perm": [0, 2, 1, 3]}), N("kt", "Transpose", ["k4"], ["kh"], {"perm": [0, 2, 3, 1]}),
        N("vt", "Transpose", ["v4"], ["vh"], {"perm": [0, 2, 1, 3]}),
        N("qk", "MatMul", ["qh", "kh"], ["s"]), N("sc", "Mul", ["s", "scale"], ["ss"]), N("sm", "Softmax", ["ss"], ["p"], {"axis": -1}),
        N("pv", "MatMul", ["p", "vh"], ["oh"]), N("ot", "Transpose", ["oh"], ["o4"], {"perm": [0, 2, 1, 3]}),
        N("or", "Reshape", ["o4", "shape_m"], ["o"]), N("proj", "MatMul", ["o", "wo"], ["y0"]), N("res", "Add", ["x", "y0"], ["y"]),
    ]
    return ox.ONNXGraph(nodes, inits, ["x"], ["y"], "block", 17)


def test_wire_roundtrip_keeps_nodes_attributes_and_tensors():
    g = _attention_block_graph()
    g2 = ox.load_onnx(ox.save_onnx(g))
    assert [n.op_type for n in g2.nodes] == [n.op_type for n in g.nodes]
    assert g2.inputs == ["x"] and g2.outputs == ["y"] and g2.opset == 17
    assert g2.nodes[0].attrs["axis"] == -1 and abs(g2.nodes[0].attrs["epsilon"] - 1e-5) < 1e-9
    assert g2.nodes[7].attrs["perm"] == [0, 2, 1, 3]
    for k, v in g.initializers.items():
        assert np.array_equal(g2.initializers[k], v) and g2.initializers[k].dtype == v.dtype


def test_summary_and_linear_extraction():
    g = _attention_block_graph()
    s = ox.summarize_graph(g.nodes)
    assert s["matmuls"] == 6 and s["layers"] == 1 and s["op_counts"]["MatMul"] == 6
    lin = ox.extract_linear_weights(g)
    assert set(lin) == {"wq", "wk", "wv", "wo"} and lin["wq"].shape == (64, 64)
    assert torch.allclose(lin["wq"], torch.from_numpy(g.initializers["wq"]).t())
    llama = [ox.ONNXOp("a", t, [], []) for t in ("Pow", "ReduceMean", "Sqrt", "Div", "MatMul", "Sigmoid", "Mul", "MatMul", "Softmax")]
    assert ox.detect_architecture(llama) == "llama"
    moe = llama + [ox.ONNXOp("t", "TopK", [], []), ox.ONNXOp("g", "Gather", [], [])]
    assert ox.detect_architecture(moe) == "moe"
    assert ox.detect_architecture([ox.ONNXOp("r", "Relu", [], [])]) == "unknown"


def test_executor_matches_pytorch_and_quantized_linears_stay_close(tmp_path):
    g = _attention_block_graph()
    path = tmp_path / "block.onnx"
    ox.save_onnx(g, path)
    x = torch.randn(2, 5, 64)
    exact = ox.ONNXExecutor.from_file(path, quantize=None)(x=x)["y"]
    # the same block in plain PyTorch
    W = {k: torch.from_numpy(v) for k, v in g.initializers.items()}
    xn = torch.nn.functional.layer_norm(x, (64,), W["ln_g"], W["ln_b"], 1e-5)
    hs = lambda t: t.view(2, 5, 4, 16).transpose(1, 2)
    q, k, v = hs(xn @ W["wq"]), hs(xn @ W["wk"]), hs(xn @ W["wv"])
    o = torch.softmax(q @ k.transpose(-1, -2) / 4.0, -1) @ v
    want = x + o.transpose(1, 2).reshape(2, 5, 64) @ W["wo"]
    assert torch.allclose(exact, want, atol=1e-5)
    qx = ox.ONNXExecutor.from_file(path, quantize="fp4", group_size=64)
    assert set(qx.linears) == {"wq", "wk", "wv", "wo"}
    approx = qx(x=x)["y"]
    assert float((approx - want).abs().max()) < 0.25 * float(want.abs().max())


def test_linear_stack_export_runs():
    ws = [torch.randn(32, 16) * 0.2, torch.randn(8, 32) * 0.2]
    bs = [torch.randn(32) * 0.1, None]
    ex = ox.ONNXExecutor(ox.load_onnx(ox.export_linear_stack(ws, bs)), quantize=None)
    x = torch.randn(3, 16)
    want = torch.relu(x @ ws[0].t() + bs[0]) @ ws[1].t()
    assert torch.allclose(ex(x=x)["h1"], want, atol=1e-5)
