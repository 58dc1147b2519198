"""Converters package surface: weight-name mapping of decoder families, activation statistics, the quantize-with-report
driver, the quantized custom operators for ONNX graphs and the NeMo entry point."""
import io
import json
import os
import tarfile

import numpy as np
import pytest
import torch
import torch.nn as nn

import metal_marlin_b200.converters as conv
from metal_marlin_b200.formats.safetensors_io import save_file
from metal_marlin_b200.models.config import get_preset

REFERENCE_CONVERTERS = [
    "CalibrationCollector", "CalibrationDataset", "CalibrationStats", "LayerReport", "MarlinFlashAttentionOp", "MarlinQuantizedLinearOp",
    "MarlinQuantizedMatMulOp", "ONNXExecutor", "ONNXGraph", "QuantizationReport", "compute_scales", "convert_nemo_to_pytorch", "create_session",
    "detect_model_type", "estimate_memory", "export_with_marlin_ops", "get_supported_architectures", "load_and_quantize", "load_config",
    "load_mapped_safetensors", "load_onnx_model", "map_weight_names", "quantize_model", "register_architecture",
]


def test_every_reference_name_resolves():
    for n in REFERENCE_CONVERTERS:
        assert getattr(conv, n) is not None, n
    assert set(REFERENCE_CONVERTERS) <= set(conv.__all__)


# ------------------------------------------------------------------------------------------------ name mapping
def _phi3_state(heads=4, kv=2, hd=8, hidden=32, inter=48):
    g = torch.Generator().manual_seed(0)
    r = lambda *s: torch.randn(*s, generator=g)     # noqa: E731
    return {"model.embed_tokens.weight": r(64, hidden), "model.final_layernorm.weight": r(hidden), "lm_head.weight": r(64, hidden),
            "model.layers.0.self_attn.qkv_proj.weight": r((heads + 2 * kv) * hd, hidden), "model.layers.0.self_attn.o_proj.weight": r(hidden, heads * hd),
            "model.layers.0.mlp.gate_up_proj.weight": r(2 * inter, hidden), "model.layers.0.mlp.down_proj.weight": r(hidden, inter),
            "model.layers.0.input_layernorm.weight": r(hidden), "model.layers.0.post_attention_layernorm.weight": r(hidden)}


def test_detect_and_map_families():
    sd = _phi3_state()
    assert conv.detect_model_type(sd.keys()) == "phi"
    m = conv.map_weight_names(sd, num_heads=4, num_kv_heads=2)
    qkv = sd["model.layers.0.self_attn.qkv_proj.weight"]
    assert torch.equal(m["model.layers.0.self_attn.q_proj.weight"], qkv[:32]) and torch.equal(m["model.layers.0.self_attn.k_proj.weight"], qkv[32:48])
    assert torch.equal(m["model.layers.0.self_attn.v_proj.weight"], qkv[48:])
    gu = sd["model.layers.0.mlp.gate_up_proj.weight"]
    assert torch.equal(m["model.layers.0.mlp.gate_proj.weight"], gu[:48]) and torch.equal(m["model.layers.0.mlp.up_proj.weight"], gu[48:])
    assert torch.equal(m["model.norm.weight"], sd["model.final_layernorm.weight"]) and "model.layers.0.self_attn.qkv_proj.weight" not in m
    with pytest.raises(ValueError):
        conv.map_weight_names(sd)                                     # fused q|k|v without head counts
    with pytest.raises(ValueError):
        conv.map_weight_names(sd, num_heads=5, num_kv_heads=2, head_dim=8)
    # head counts from a config dict
    m2 = conv.map_weight_names(sd, config={"num_attention_heads": 4, "num_key_value_heads": 2})
    assert set(m2) == set(m)
    phi2 = {"transformer.embd.wte.weight": torch.zeros(8, 4), "transformer.h.3.mixer.Wqkv.weight": torch.arange(48.).reshape(12, 4),
            "transformer.h.3.mixer.Wqkv.bias": torch.arange(12.), "transformer.h.3.mlp.fc1.weight": torch.zeros(16, 4),
            "transformer.h.3.mlp.fc2.weight": torch.zeros(4, 16), "lm_head.ln.weight": torch.ones(4)}
    assert conv.detect_model_type(phi2) == "phi2"
    m = conv.map_weight_names(phi2, num_heads=2)
    assert m["model.layers.3.self_attn.k_proj.bias"].tolist() == [4., 5., 6., 7.] and "model.layers.3.mlp.up_proj.weight" in m
    assert m["model.norm.weight"].shape == (4,) and "model.embed_tokens.weight" in m
    assert conv.detect_model_type({"model.layers.0.mlp.c_fc.weight"}) == "starcoder2"
    assert conv.detect_model_type({"model.layers.0.self_attn.q_proj.bias", "lm_head.weight"}) == "qwen2"
    assert conv.detect_model_type({"model.embed_tokens.weight", "model.layers.0.self_attn.q_proj.weight"}) == "gemma"
    assert conv.detect_model_type({"model.embed_tokens.weight", "lm_head.weight"}) == "llama"
    sc = conv.map_weight_names({"model.layers.1.mlp.c_fc.weight": torch.zeros(8, 4), "model.layers.1.mlp.c_proj.bias": torch.zeros(4)}, "starcoder2")
    assert set(sc) == {"model.layers.1.mlp.up_proj.weight", "model.layers.1.mlp.down_proj.bias"}


def test_register_architecture():
    assert {"llama", "mistral", "phi", "phi2", "qwen2", "gemma", "starcoder2"} <= set(conv.get_supported_architectures())
    rules = [("gpt.blocks.{layer}.attn.fused.weight", "model.layers.{layer}.self_attn|weight", "qkv"),
             ("gpt.blocks.{layer}.ff.out.weight", "model.layers.{layer}.mlp.down_proj.weight")]
    conv.register_architecture("toy-gpt", rules, overwrite=True)
    with pytest.raises(ValueError):
        conv.register_architecture("toy-gpt", rules)
    m = conv.map_weight_names({"gpt.blocks.7.attn.fused.weight": torch.zeros(12, 4), "gpt.blocks.7.ff.out.weight": torch.zeros(4, 8), "other": torch.zeros(1)},
                              "toy-gpt", num_heads=2, num_kv_heads=2)
    assert set(m) == {"model.layers.7.self_attn.q_proj.weight", "model.layers.7.self_attn.k_proj.weight", "model.layers.7.self_attn.v_proj.weight",
                      "model.layers.7.mlp.down_proj.weight", "other"}
    with pytest.raises(KeyError):
        conv.map_weight_names({"other": torch.zeros(1)}, "toy-gpt", strict=True)
    with pytest.raises(ValueError):
        conv.map_weight_names({}, "no-such-family")


def _float_checkpoint(path):
    import metal_marlin_b200.quant as q
    cfg = get_preset("tiny-llama")
    os.makedirs(path)
    save_file(q.random_hf_state(cfg, 0), os.path.join(path, "model.safetensors"), metadata={"format": "pt"})
    cfg.save_pretrained(path)
    return cfg


def test_estimate_load_and_quantize(tmp_path):
    src = str(tmp_path / "hf")
    cfg = _float_checkpoint(src)
    assert conv.load_config(src).hidden_size == cfg.hidden_size and conv.load_config(os.path.join(src, "config.json")).vocab_size == cfg.vocab_size
    est = conv.estimate_memory(src, group_size=64)
    assert 0 < est["quantized_elements"] < est["total_elements"] and est["quantized_gb"] < est["fp16_gb"] and est["savings_ratio"] > 1.5
    sd, c2 = conv.load_mapped_safetensors(src)
    assert c2.num_hidden_layers == cfg.num_hidden_layers and "model.layers.0.self_attn.q_proj.weight" in sd
    q, _ = conv.load_and_quantize(src, "int4", group_size=64)
    from metal_marlin_b200.quant import QuantizedTensor, dequantize
    w = sd["model.layers.0.mlp.down_proj.weight"].float()
    qt = q["model.layers.0.mlp.down_proj.weight"]
    assert isinstance(qt, QuantizedTensor) and not isinstance(q["model.embed_tokens.weight"], QuantizedTensor)
    assert float((dequantize(qt).float() - w).norm() / w.norm()) < 0.15


def test_quantize_model_report(tmp_path):
    src, dst = str(tmp_path / "hf"), str(tmp_path / "q")
    _float_checkpoint(src)
    rep = conv.quantize_model(src, dst, group_size=64, skip_layers=["down_proj"])
    assert rep.num_quantized > 0 and rep.total_tensors == rep.num_quantized + rep.num_skipped and len(rep.layers) == rep.num_quantized
    assert all("down_proj" not in r.name for r in rep.layers) and all(r.snr_db > 10 and r.rms_error > 0 and r.max_error >= r.rms_error for r in rep.layers)
    assert rep.avg_snr_db > 10 and rep.output_size_mb > 0
    with open(os.path.join(dst, "quantization_report.json")) as f:
        d = json.load(f)
    assert d["num_quantized"] == rep.num_quantized and len(d["layers"]) == len(rep.layers)
    from metal_marlin_b200.models.mmfp4_causal_lm import MMFP4ForCausalLM
    lm = MMFP4ForCausalLM.from_pretrained(dst, "cpu")
    assert torch.isfinite(lm.forward_logits([1, 2, 3, 4]).float()).all()
    with pytest.raises(ValueError):
        conv.quantize_model(src, str(tmp_path / "q2"), quant_type="int3")


def test_quantize_model_with_calibration_tokens(tmp_path):
    src, dst = str(tmp_path / "hf"), str(tmp_path / "q")
    cfg = _float_checkpoint(src)
    g = torch.Generator().manual_seed(0)
    calib = [torch.randint(0, cfg.vocab_size, (24,), generator=g) for _ in range(3)]
    rep = conv.quantize_model(src, dst, calibration_data=calib, group_size=64)
    assert rep.num_quantized > 0 and rep.avg_snr_db > 8


# ------------------------------------------------------------------------------------------------ activation statistics
def test_calibration_dataset(tmp_path, monkeypatch):
    p = tmp_path / "calib.txt"
    p.write_text("first paragraph\nstill first\n\nsecond one\n\n\nthird")
    ds = conv.CalibrationDataset.from_file(str(p))
    assert len(ds) == 3 and ds.name == "calib" and ds[1] == "second one"
    assert len(conv.CalibrationDataset.from_file(str(p), max_samples=2)) == 2
    ds2 = conv.CalibrationDataset.from_texts(["a b", "c"], name="mine")
    assert ds2.name == "mine" and list(ds2) == ["a b", "c"]

    class Tok:
        def encode(self, t):
            return [ord(c) for c in t]
    enc = ds2.tokenize(Tok(), max_length=4)
    assert enc[0]["input_ids"].tolist() == [[97, 32, 98, 0]] and enc[1]["attention_mask"].tolist() == [[1, 0, 0, 0]]
    monkeypatch.setenv("MMB200_CALIBRATION_DIR", str(tmp_path))
    with pytest.raises(FileNotFoundError):
        conv.CalibrationDataset.bartowski_v3(cache_dir=str(tmp_path / "none"))
    (tmp_path / "calibration_datav3.txt").write_text("a sample that is long enough\n\nanother sample that is long enough")
    assert len(conv.CalibrationDataset.bartowski_v3()) == 2


@pytest.mark.parametrize("method", ["histogram", "exact"])
def test_collector_percentiles_and_scales(method):
    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(16, 32), nn.ReLU(), nn.Linear(32, 8))
    col = conv.CalibrationCollector(model, percentile_low=1.0, percentile_high=99.0, method=method, num_bins=4096)
    assert col.num_layers == 2
    xs = [torch.randn(256, 16) * (1 + i) for i in range(4)]          # growing range exercises the range doubling
    for x in xs:
        model(x)
    stats = col.get_stats()
    s0 = stats["0"]
    allx = torch.cat(xs).reshape(-1)
    assert s0.num_batches == 4 and float(s0.min_val) == float(allx.min()) and float(s0.absmax) == float(allx.abs().max())
    lo, hi = torch.quantile(allx, 0.01), torch.quantile(allx, 0.99)
    assert abs(float(s0.percentile_low) - float(lo)) < 0.05 * float(lo.abs()) and abs(float(s0.percentile_high) - float(hi)) < 0.05 * float(hi)
    assert float(stats["2"].min_val) >= 0                              # input of the second Linear is a ReLU output
    sc = conv.compute_scales(stats, "fp4")
    assert sc["0"][1] is None and abs(float(sc["0"][0]) - max(abs(float(s0.percentile_low)), float(s0.percentile_high)) / 6) < 1e-6
    assert float(conv.compute_scales(stats, "fp4", use_percentile=False)["0"][0]) == pytest.approx(float(s0.absmax) / 6)
    scale, zero = conv.compute_scales(stats, "int4_asym")["2"]
    assert 0 <= float(zero) <= 15 and float(scale) > 0
    with pytest.raises(ValueError):
        conv.compute_scales(stats, "int5")
    col.remove_hooks()
    model(xs[0])
    assert col.get_stats()["0"].num_batches == 4
    col.reset()
    assert col.stats == {}
    only = conv.CalibrationCollector(model, layers_to_calibrate=["2"])
    assert only.num_layers == 1
    with pytest.raises(ValueError):
        conv.CalibrationCollector(model, method="sketch")


# ------------------------------------------------------------------------------------------------ custom operators
def test_custom_ops_rewrite_and_session(tmp_path):
    from metal_marlin_b200.compat_api import pack_fp4_weights, unpack_fp4_weights
    from metal_marlin_b200.converters import onnx as ox
    torch.manual_seed(0)
    ws = [torch.randn(256, 128) * 0.1, torch.randn(64, 256) * 0.1]
    bs = [torch.randn(256) * 0.1, None]
    src = tmp_path / "mlp.onnx"
    ox.export_linear_stack(ws, bs, path=src)
    out = tmp_path / "mlp_q.onnx"
    conv.export_with_marlin_ops(src, out, None, group_size=128)
    g = conv.load_onnx_model(out)
    assert [(n.op_type, n.domain) for n in g.nodes] == [("MarlinQuantizedLinear", "com.metal_marlin"), ("Relu", ""), ("MarlinQuantizedMatMul", "com.metal_marlin")]
    assert g.initializers["w0_packed"].dtype == np.uint32 and "w0" not in g.initializers and g.opset == 17
    assert os.path.getsize(out) < 0.45 * os.path.getsize(src)
    sess = conv.create_session(out)
    assert [a.name for a in sess.get_inputs()] == ["x"]
    x = np.random.RandomState(0).randn(4, 128).astype(np.float32)
    y = sess.run(None, {"x": x})[0]
    dq = []
    for w in ws:
        p, sc, meta = pack_fp4_weights(w.t().contiguous().numpy(), 128)
        dq.append(torch.from_numpy(unpack_fp4_weights(p, sc, meta).astype(np.float32)))
    ref = torch.relu(torch.from_numpy(x) @ dq[0] + bs[0]) @ dq[1]
    assert float((torch.from_numpy(y) - ref).norm() / ref.norm()) < 0.02
    # explicit weights for one MatMul only
    p, sc, _ = pack_fp4_weights(ws[1].t().contiguous().numpy(), 128)
    g2 = ox.load_onnx(conv.export_with_marlin_ops(src, None, {"w1": (p, sc)}, group_size=128))
    assert [n.op_type for n in g2.nodes] == ["MatMul", "Add", "Relu", "MarlinQuantizedMatMul"]
    with pytest.raises(FileNotFoundError):
        conv.create_session(out, custom_lib_path=str(tmp_path / "missing.so"))
    # operator definitions
    A = x[:3].astype(np.float16)
    p0, sc0, _ = pack_fp4_weights(ws[0].t().contiguous().numpy(), 128)
    o = conv.MarlinQuantizedMatMulOp.compute(A, p0, sc0, group_size=128)
    assert o.dtype == np.float16 and np.abs(o.astype(np.float32) - A.astype(np.float32) @ dq[0].numpy()).max() < 0.05
    ol = conv.MarlinQuantizedLinearOp.compute(A, p0, sc0, bs[0].numpy().astype(np.float16), group_size=128)
    assert np.abs(ol.astype(np.float32) - o.astype(np.float32) - bs[0].numpy()).max() < 0.02
    Q = np.random.RandomState(1).randn(1, 2, 8, 16).astype(np.float16)
    oa = conv.MarlinFlashAttentionOp.compute(Q, Q, Q, causal=1)
    ref = torch.nn.functional.scaled_dot_product_attention(*(torch.from_numpy(Q).float(),) * 3, is_causal=True)
    assert np.abs(oa.astype(np.float32) - ref.numpy()).max() < 0.03
    assert conv.MarlinQuantizedMatMulOp.get_inputs()[1] == ("B_packed", "tensor(uint32)") and "group_size" in conv.MarlinQuantizedLinearOp.get_attrs()
    assert conv.MarlinFlashAttentionOp.get_outputs() == [("O", "tensor(float16)")]


# ------------------------------------------------------------------------------------------------ NeMo
def test_convert_nemo_to_pytorch(tmp_path):
    import yaml
    heads, kv, hd, hidden, ffn = 4, 2, 8, 32, 48
    sd = {"model.embedding.word_embeddings.weight": torch.randn(64, hidden),
          "model.decoder.layers.0.self_attention.linear_qkv.weight": torch.randn((heads + 2 * kv) * hd, hidden),
          "model.decoder.layers.0.self_attention.linear_proj.weight": torch.randn(hidden, heads * hd),
          "model.decoder.layers.0.mlp.linear_fc1.weight": torch.randn(2 * ffn, hidden),
          "model.decoder.layers.0.mlp.linear_fc2.weight": torch.randn(hidden, ffn),
          "model.decoder.final_layernorm.weight": torch.ones(hidden), "model.output_layer.weight": torch.randn(64, hidden)}
    cfg = {"num_attention_heads": heads, "num_query_groups": kv, "hidden_size": hidden, "num_layers": 1, "ffn_hidden_size": ffn, "kv_channels": hd,
           "activation": "fast-swiglu", "vocab_size": 64}
    nemo = tmp_path / "m.nemo"
    with tarfile.open(nemo, "w") as tf:
        for name, data in (("model_config.yaml", yaml.safe_dump(cfg).encode()), ("model_weights.ckpt", None)):
            if data is None:
                buf = io.BytesIO()
                torch.save(sd, buf)
                data = buf.getvalue()
            ti = tarfile.TarInfo(name)
            ti.size = len(data)
            tf.addfile(ti, io.BytesIO(data))
    only = conv.convert_nemo_to_pytorch(str(nemo), str(tmp_path / "x"), extract_config_only=True, config_output=str(tmp_path / "cfg" / "c.json"))
    assert only["output"] is None and only["config"]["num_key_value_heads"] == kv and os.path.isfile(tmp_path / "cfg" / "c.json")
    info = conv.convert_nemo_to_pytorch(str(nemo), str(tmp_path / "out"))
    assert info["output"].endswith("model.safetensors") and info["num_tensors"] >= 8 and os.path.isfile(tmp_path / "out" / "config.json")
    from metal_marlin_b200.formats.safetensors_io import SafetensorsFile
    names = set(SafetensorsFile(info["output"]).keys())
    assert {"model.layers.0.self_attn.q_proj.weight", "model.layers.0.mlp.gate_proj.weight", "model.layers.0.mlp.down_proj.weight"} <= names
    pt = conv.convert_nemo_to_pytorch(str(nemo), str(tmp_path / "w.pt"), use_safetensors=False)
    assert set(torch.load(pt["output"], weights_only=True)) == names
    with pytest.raises(FileNotFoundError):
        conv.convert_nemo_to_pytorch(str(tmp_path / "none.nemo"), str(tmp_path / "o"))
    with pytest.raises(ValueError):
        conv.convert_nemo_to_pytorch(str(tmp_path / "cfg" / "c.json"), str(tmp_path / "o"))
