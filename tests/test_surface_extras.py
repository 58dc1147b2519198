"""FLOP calculator, GEMM operation objects, mixed-format model packing, visualization, native dispatch wrapper and the
graph-captured decoder layer."""
import json
import math
import os

import numpy as np
import pytest
import torch
import torch.nn as nn


# ------------------------------------------------------------------------------------------------ FLOPs
def test_flops_calculator():
    from metal_marlin_b200.models.config import get_preset
    from metal_marlin_b200.utils import (LayerFLOPsCalculator, calculate_layer_flops, estimate_marlin_linear_flops, profile_model_layers)
    assert estimate_marlin_linear_flops(64, 32, 2, 3, quantized=False, include_bias=False) == 2 * 6 * 64 * 32
    assert estimate_marlin_linear_flops(64, 32, 2, 3, quantized=False, include_bias=True) == 2 * 6 * 64 * 32 + 6 * 32
    assert estimate_marlin_linear_flops(64, 32, 1, 300, quantized=True, include_bias=False) == 2 * 300 * 64 * 32 + 3 * 64 * 32
    assert calculate_layer_flops("linear", in_features=64, out_features=32, batch_size=2, seq_len=3, quantized=False) == 2 * 6 * 64 * 32
    assert calculate_layer_flops("attention", batch_size=1, seq_len=8, num_heads=2, head_dim=4) == 4 * 2 * 64 * 4 + 5 * 2 * 64
    assert calculate_layer_flops("layernorm", batch_size=2, seq_len=4, hidden_dim=16) == 5 * 8 * 16 and calculate_layer_flops("embedding") == 0
    with pytest.raises(ValueError):
        calculate_layer_flops("conv3d")
    model = nn.Sequential(nn.Embedding(10, 16), nn.Linear(16, 32), nn.LayerNorm(32), nn.Linear(32, 8, bias=False))
    calc = profile_model_layers(model, batch_size=2, seq_len=5, quantized=False)
    assert [r.module_type for r in calc.get_results()] == ["Embedding", "Linear", "LayerNorm", "Linear"]
    assert calc.get_layer("1").flops == 2 * 10 * 16 * 32 + 10 * 32 and calc.get_layer("3").flops == 2 * 10 * 32 * 8
    assert calc.total_params == sum(p.numel() for p in model.parameters()) and calc.total_tflops == calc.total_flops / 1e12
    assert calc.add_module("x", nn.ReLU()) is None and "GFLOP" in calc.summary_text(2)
    r = LayerFLOPsCalculator().add_module("lin", nn.Linear(8, 4), input_shape=(3, 7, 8))
    assert r.flops == 2 * 21 * 8 * 4 + 21 * 4 and r.gflops == r.flops / 1e9
    from metal_marlin_b200.layers import MMFP4Linear
    q = LayerFLOPsCalculator(1, 1).add_module("q", MMFP4Linear.from_float(torch.randn(32, 128), group_size=64, device="cpu"))
    assert q.metadata["quantized"] and q.flops == 2 * 128 * 32 + 128 * 32
    cfg = get_preset("glm-4.7-flash")
    c = profile_model_layers(cfg, 1, 1, quantized=False)
    active = cfg.param_count()["active"]
    assert 0.98 < c.total_flops / (2 * active) < 1.05                      # decode FLOPs are twice the active parameters plus a little
    assert c.get_layer("layers.0.mlp") is not None and c.get_layer("layers.1.moe.routed").metadata["experts_per_token"] == cfg.num_experts_per_tok
    calc.clear()
    assert calc.total_flops == 0


# ------------------------------------------------------------------------------------------------ GEMM objects
def test_gemm_operation_objects():
    import metal_marlin_b200.ops as ops
    from metal_marlin_b200.compat_api import pack_fp4_weights, unpack_fp4_weights
    torch.manual_seed(0)
    w = torch.rand(256, 64) * 2 - 1
    p = ops.pack_int8_weights(w)
    q = ops.unpack_int8_weights(p, 256)
    assert p.shape == (64, 64) and p.dtype == torch.int32 and torch.equal(q.float(), torch.clamp(torch.round(w * 127), -128, 127))
    assert ops.pack_int8_weights(w[:254]).shape == (64, 64) and torch.equal(ops.unpack_int8_weights(ops.pack_int8_weights(w[:254]), 254), q[:254])
    scales = torch.full((4, 64), 1 / 127.0)
    x = torch.randn(5, 256)
    g8 = ops.GemmInt8()
    ref = x @ (q.float() / 127)
    assert float((g8(x, p, scales, None, 64) - ref).norm() / ref.norm()) < 5e-3
    zeros = torch.full((4, 64), 3.0)
    ref_z = x @ ((q.float() - 3) / 127)
    assert float((ops.GemmInt8().forward(x, p, scales, zeros, 64) - ref_z).norm() / ref_z.norm()) < 5e-3
    W = torch.randn(128, 32) * 0.1
    pk, sc, meta = pack_fp4_weights(W.numpy(), 64, output_backend="torch")
    g4 = ops.GemmFp4()
    x4 = torch.randn(2, 3, 128)
    y = g4(x4, pk, sc, 64)
    ref4 = x4 @ torch.from_numpy(unpack_fp4_weights(pk.numpy(), sc.numpy(), meta).astype(np.float32))
    assert y.shape == (2, 3, 32) and float((y - ref4).norm() / ref4.norm()) < 0.02
    g4(x4, pk, sc, 64)
    assert len(g4._cache) == 1                                              # the device weight of a packed tensor is built once
    assert ops.MetalQuantizedLinear is not None
    with pytest.raises(AttributeError):
        ops.no_such_name


# ------------------------------------------------------------------------------------------------ mixed-format model
def test_mixed_format_model_roundtrip(tmp_path):
    import metal_marlin_b200.converters as conv
    from metal_marlin_b200.compat_api import Precision
    torch.manual_seed(0)
    weights = {"a.weight": torch.randn(32, 128), "b.weight": torch.randn(16, 96).numpy(), "norm.weight": torch.ones(128), "c.weight": torch.randn(8, 64)}
    pmap = {"a.weight": (Precision.FP4, 64), "b.weight": (Precision.INT8, 64), "c.weight": (Precision.BF16, 0)}
    out = str(tmp_path / "m" / "model.safetensors")
    h = conv.pack_mixed_format_model(weights, pmap, out)
    assert h.layer_formats["a.weight"] == "fp4" and h.layer_group_sizes["b.weight"] == 32 and h.layer_formats["norm.weight"] == "bf16"
    assert h.total_params == 32 * 128 + 16 * 96 + 128 + 8 * 64 and h.quantized_params == 32 * 128 + 16 * 96 and 4 < h.average_bits < 8
    assert "x fp4" in h.summary() and conv.MixedFormatHeader.from_json(h.to_json()) == h
    tensors, h2 = conv.load_mixed_format_model(out)
    assert h2 == h and "a.weight.scales" in tensors and tensors["c.weight"].dtype == torch.bfloat16
    assert h2.get_format("a.weight.scales") == "fp4" and h2.get_group_size("a.weight") == 64 and h2.get_format("zzz") is None
    assert conv.get_layer_precision(h2, "b.weight") == (Precision.INT8, 32) and conv.get_layer_precision(h2, "zzz") == (Precision.FP16, 0)
    back = conv.MixedFormatPack.load(out)
    assert float((back.dequantize("a.weight") - weights["a.weight"]).norm() / weights["a.weight"].norm()) < 0.15
    other = str(tmp_path / "m" / "second.safetensors")
    conv.pack_mixed_format_model({"d.weight": torch.randn(8, 64)}, {"d.weight": (Precision.INT4, 32)}, other)
    hm = conv.merge_mixed_format_models([out, other], str(tmp_path / "m" / "merged.safetensors"))
    assert set(hm.layer_formats) == set(h.layer_formats) | {"d.weight"} and hm.total_params == h.total_params + 8 * 64
    with pytest.raises(ValueError):
        conv.merge_mixed_format_models([out, out], str(tmp_path / "m" / "dup.safetensors"))
    with pytest.raises(FileNotFoundError):
        conv.load_mixed_format_model(str(tmp_path / "none.safetensors"))
    from metal_marlin_b200.formats.safetensors_io import save_file
    plain = str(tmp_path / "plain.safetensors")
    save_file({"x": torch.zeros(2)}, plain)
    with pytest.raises(ValueError):
        conv.load_mixed_format_model(plain)


# ------------------------------------------------------------------------------------------------ visualization
def test_error_metrics_and_analyzer():
    from metal_marlin_b200.visualization import ErrorAnalyzer, ErrorMetrics
    torch.manual_seed(0)
    o = torch.randn(64, 64)
    q = o + 0.01 * torch.randn(64, 64)
    m = ErrorMetrics.from_tensors(o, q.numpy(), bits_per_weight=4.25)
    e = (q - o).double()
    assert m.mse == pytest.approx(float(e.pow(2).mean())) and m.rmse == pytest.approx(math.sqrt(m.mse)) and m.mae == pytest.approx(float(e.abs().mean()))
    assert m.snr == pytest.approx(10 * math.log10(float(o.double().pow(2).mean()) / m.mse)) and m.psnr > m.snr
    assert m.cosine_similarity > 0.999 and m.correlation > 0.999 and m.compression_ratio == pytest.approx(16 / 4.25) and abs(m.quantization_kurtosis) < 0.5
    assert 0 < m.outlier_ratio < 0.2 and set(m.to_dict()) >= {"mse", "psnr", "outlier_ratio"}
    same = ErrorMetrics.from_tensors(o, o)
    assert same.mse == 0 and same.snr == float("inf") and same.cosine_similarity == pytest.approx(1.0)
    with pytest.raises(ValueError):
        ErrorMetrics.from_tensors(o, o[:3])
    an = ErrorAnalyzer()
    for i, noise in enumerate((0.01, 0.05, 0.02)):
        an.add_layer_metrics(f"l{i}", "fp4", ErrorMetrics.from_tensors(o, o + noise * torch.randn(64, 64), 4.25))
        an.add_layer_metrics(f"l{i}", "int8", ErrorMetrics.from_tensors(o, o + noise / 10 * torch.randn(64, 64), 8.25))
    assert an.formats() == ["fp4", "int8"] and set(an.get_layer_comparison("l1")) == {"fp4", "int8"} and an.get_layer_comparison("zz") is None
    s = an.get_format_summary("fp4")
    assert s["num_layers"] == 3 and s["max_rmse"] == pytest.approx(an.layer_metrics["l1"]["fp4"].rmse) and an.get_format_summary("nf4") == {}
    assert an.get_best_format_per_layer("rmse")["l0"][0] == "int8" and an.get_best_format_per_layer("snr")["l0"][0] == "int8"
    assert [l for l, _ in an.identify_problematic_layers("fp4")] == ["l1", "l2", "l0"] and an.identify_problematic_layers("fp4", threshold_rmse=0.03, top_k=5)[0][0] == "l1"
    assert len(an.identify_problematic_layers("fp4", threshold_rmse=0.03)) == 1 and set(an.to_dict()) == {"layers", "formats"}


def test_weight_visualizer_and_plots(tmp_path):
    from metal_marlin_b200.formats.safetensors_io import save_file
    from metal_marlin_b200.visualization import (WeightVisualizer, plot_error_distribution, plot_error_heatmap, plot_layer_errors, plot_weight_comparison)
    torch.manual_seed(0)
    ws = {f"model.layers.{i}.mlp.up_proj.weight": torch.randn(64, 128) * (0.02 * (i + 1)) for i in range(4)}
    ws["model.norm.weight"] = torch.ones(128)
    ws["model.layers.0.idx"] = torch.zeros(4, 4, dtype=torch.int32)
    f = str(tmp_path / "model.safetensors")
    save_file(ws, f)
    viz = WeightVisualizer.from_safetensors(f, group_size=64)
    assert len(viz.layer_names()) == 4 and len(WeightVisualizer.from_safetensors(str(tmp_path), max_tensors=2).layer_names()) == 2
    assert WeightVisualizer.from_safetensors(f, name_filter="layers.3").layer_names() == ["model.layers.3.mlp.up_proj.weight"]
    name = "model.layers.1.mlp.up_proj.weight"
    m4, m8 = viz.compare_quantization(name, "fp4"), viz.compare_quantization(name, "int8")
    assert m8.rmse < m4.rmse and m4.bits_per_weight == 4.25 and 15 < m4.snr < 25
    assert set(viz.compare_formats(name, ("int4", "nf4"))) == {"int4", "nf4"}
    with pytest.raises(KeyError):
        viz.compare_quantization("nope", "fp4")
    with pytest.raises(ValueError):
        viz.compare_quantization(name, "fp5")
    rep = viz.generate_error_report(str(tmp_path / "rep"), ("fp4", "int8"), plots_for_worst=1)
    files = set(os.listdir(tmp_path / "rep"))
    assert {"error_report.json", "layer_errors_fp4.png", "layer_errors_int8.png", "heatmap_model_layers_3_mlp_up_proj_weight_fp4.png",
            "compare_model_layers_3_mlp_up_proj_weight_fp4.png"} <= files
    assert json.load(open(tmp_path / "rep" / "error_report.json"))["problematic_layers"]["fp4"][0][0] == "model.layers.3.mlp.up_proj.weight"
    assert rep["formats"]["int8"]["mean_snr"] > rep["formats"]["fp4"]["mean_snr"] and rep["best_format_per_layer"][name]["format"] == "int8"
    o = ws[name]
    q = viz.quantize(name, "fp4")
    hm = plot_error_heatmap(o, q, str(tmp_path / "p" / "h.png"), title="t")
    assert hm.shape == (64 + 16, 128, 3) and hm.dtype == np.uint8 and os.path.getsize(tmp_path / "p" / "h.png") > 0
    big = plot_error_heatmap(torch.randn(300, 1000), torch.randn(300, 1000), max_side=100)
    assert big.shape[0] <= 100 and big.shape[1] <= 100
    exact = plot_error_heatmap(o, o)
    assert (exact == 255).all()                                             # zero error is white
    cmp_img = plot_weight_comparison(o, q)
    assert cmp_img.shape == (64 + 16, 3 * 128 + 12, 3)
    d1 = plot_error_distribution(q - o, title="fp4")
    d2 = plot_error_distribution({"fp4": q - o, "int8": viz.quantize(name, "int8") - o}, str(tmp_path / "p" / "d.png"), log=False)
    assert d1.shape == d2.shape == (360, 640, 3) and (d1 != 255).any() and (d2 != 255).any()
    bars = plot_layer_errors({f"l{i}": float(i) for i in range(10)}, highlight_top=2)
    assert bars.shape == (360, 800, 3) and ((bars == np.array([210, 60, 50])).all(-1)).any() and ((bars == np.array([40, 90, 200])).all(-1)).any()
    assert plot_layer_errors({}).shape == (360, 800, 3)
    assert viz.plot_error_distribution(name, ("fp4", "int4")).shape == (360, 640, 3)


# ------------------------------------------------------------------------------------------------ dispatch wrapper, traced layer
def test_native_dispatch_wrapper_on_cpu():
    from metal_marlin_b200.serving import ServingCppDispatcher, ServingCppEngineWrapper, create_serving_cpp_dispatcher
    d = ServingCppDispatcher("cpu")
    assert d.available is False and create_serving_cpp_dispatcher("cpu") is None
    with pytest.raises(RuntimeError):
        d.dispatch_sync("rmsnorm", torch.zeros(1))
    assert d.dispatch_sync(lambda a, b=1: a + b, 2, b=3) == 5
    h = d.dispatch_async(torch.add, torch.ones(2), torch.ones(2))
    assert d.is_complete(h) and torch.equal(d.wait(h), torch.full((2,), 2.0))
    m = d.get_metrics()
    assert m["sync_dispatches"] == 1 and m["async_dispatches"] == 1 and m["total_dispatches"] == 2 and m["waits"] == 1 and m["avg_host_launch_us"] > 0
    d.reset_metrics()
    assert d.get_metrics()["total_dispatches"] == 0
    w = ServingCppEngineWrapper(dispatcher=d)
    assert w.available is False and w.dispatch_for_decode(lambda: 7) == 7 and w.wait(w.dispatch_for_prefill(lambda: 8)) == 8
    assert w.get_metrics()["decode_calls"] == 1 and w.get_metrics()["prefill_calls"] == 1


def test_traced_decoder_layer_eager_path():
    from metal_marlin_b200.engine.traced import TracedDecoderLayer
    lin = nn.Linear(16, 16)
    calls = []

    def layer(h, scale=None):
        calls.append(1)
        return (lin(h) * scale, None)
    s = torch.tensor(2.0)
    t = TracedDecoderLayer(layer, batch_size=2, seq_len=3, hidden_size=16, dtype=torch.float32, device="cpu")
    x = torch.randn(2, 3, 16)
    y = t(x, scale=s)
    assert torch.allclose(y, lin(x) * 2) and t.shape == (2, 3, 16) and t.replays == 0
    s.fill_(3.0)                                                            # tensors bound at compile are read at call time
    assert torch.allclose(t(x, scale=s), lin(x) * 3)
    with pytest.raises(ValueError):
        t(torch.randn(1, 3, 16))
    with pytest.raises(ValueError):
        t(x, scale=torch.tensor(1.0))


@pytest.mark.gpu
def test_traced_decoder_layer_graph_replay_gpu():
    from metal_marlin_b200.engine.traced import TracedDecoderLayer
    from metal_marlin_b200.serving import ServingCppDispatcher
    torch.manual_seed(0)
    lin = nn.Linear(64, 64).cuda().bfloat16()
    t = TracedDecoderLayer(lambda h: torch.nn.functional.silu(lin(h)) + h, 1, 4, 64)
    for _ in range(3):
        x = torch.randn(1, 4, 64, device="cuda", dtype=torch.bfloat16)
        ref = torch.nn.functional.silu(lin(x)) + x
        assert torch.allclose(t(x).float(), ref.float(), atol=0.1, rtol=2e-2)          # the library GEMM may pick another algorithm under capture
    assert t.replays == 3
    d = ServingCppDispatcher()
    assert d.available
    x = torch.randn(8, 64, device="cuda", dtype=torch.bfloat16)
    h = d.dispatch_async(torch.add, x, x)
    assert torch.equal(d.wait(h), x + x) and d.is_complete(h)
    assert torch.equal(d.dispatch_sync(torch.mul, x, 2), x * 2)


# ------------------------------------------------------------------------------------------------ transient buffer, ranges, activations
def test_transient_buffer():
    from metal_marlin_b200.memory import TransientBufferCPP, get_transient_buffer_cpp, reset_transient_buffer_cpp, transient_buffer_cpp_stats
    reset_transient_buffer_cpp()
    assert transient_buffer_cpp_stats("cpu") is None
    buf = get_transient_buffer_cpp("cpu", 4096)
    assert buf is get_transient_buffer_cpp("cpu", 1024) and TransientBufferCPP.is_available() and not buf.is_cpp_backend
    slab, off0 = buf.allocate(100)
    _, off1 = buf.allocate_bytes(10)
    assert off0 == 0 and off1 == 256 and slab.numel() == 4096 and buf.used == 266 and buf.available == 4096 - 266
    t = buf.tensor((4, 8), torch.float32)
    t.fill_(1.5)
    assert t.data_ptr() == slab.data_ptr() + 512 and buf.utilization == pytest.approx((512 + 128) / 4096)
    with pytest.raises(MemoryError):
        buf.allocate(4096)
    buf.reset()
    assert buf.used == 0 and buf.stats()["resets"] == 1 and buf.stats()["high_water"] == 640 and buf.stats()["allocations"] == 3
    assert get_transient_buffer_cpp("cpu", 8192) is not buf and transient_buffer_cpp_stats("cpu")["capacity"] == 8192
    reset_transient_buffer_cpp()


def test_activation_ranges_and_scales(tmp_path):
    import metal_marlin_b200 as mm
    from metal_marlin_b200.converters import CalibrationDatasetLoader
    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(8, 16), nn.ReLU(), nn.Linear(16, 4))
    xs = [torch.randn(5, 8) * (i + 1) for i in range(3)]
    r = mm.compute_activation_ranges(model, xs)
    allx = torch.cat(xs)
    assert r["0"] == (pytest.approx(float(allx.min())), pytest.approx(float(allx.max()))) and r["2"][0] >= 0
    assert set(mm.compute_activation_ranges(model, xs, layers=["2"])) == {"2"}
    s = mm.ranges_to_scales({"a": (-3.0, 6.0), "b": (-1.0, 0.5)}, "fp4")
    assert s == {"a": 1.0, "b": pytest.approx(1 / 6)} and mm.ranges_to_scales({"a": (-3.0, 6.0)}, "int4_asym")["a"] == pytest.approx(0.6)
    assert mm.ranges_to_scales({"a": (-3.0, 6.0)}, "int8_sym")["a"] == pytest.approx(6 / 127) and mm.ranges_to_scales({"a": (0.0, 0.0)}, "int4_sym")["a"] > 0
    with pytest.raises(ValueError):
        mm.ranges_to_scales({"a": (0, 1)}, "fp3")
    p = str(tmp_path / "r" / "ranges.json")
    mm.save_ranges(r, p)
    assert mm.load_ranges(p) == {k: (float(a), float(b)) for k, (a, b) in r.items()}
    # an engine model: ranges per checkpoint tensor through the capture hook
    from metal_marlin_b200.formats.safetensors_io import save_file
    from metal_marlin_b200.models.config import get_preset
    from metal_marlin_b200.models.mmfp4_causal_lm import MMFP4ForCausalLM
    import metal_marlin_b200.quant as q
    cfg = get_preset("tiny-llama")
    d = str(tmp_path / "ck")
    q.save_random_checkpoint(cfg, d, seed=0)
    lm = MMFP4ForCausalLM.from_pretrained(d, "cpu")
    er = mm.compute_activation_ranges(lm, [[1, 2, 3, 4, 5], [7, 8, 9]])
    assert any(k.endswith("q_proj.weight") for k in er) and all(lo <= hi for lo, hi in er.values())
    assert set(mm.compute_activation_ranges(lm, [[1, 2, 3]], layers=["down_proj"])) == {k for k in er if "down_proj" in k}
    with pytest.raises(ValueError):
        mm.compute_activation_ranges(lm, ["some text"])
    f = tmp_path / "calib.txt"
    f.write_text("x" * 120 + "\n\n" + "short\n\n" + "y" * 150)
    assert len(CalibrationDatasetLoader.from_file(str(f), min_sample_length=100)) == 2
    (tmp_path / "calibration_datav3.txt").write_text("x" * 120 + "\n\n" + "a sample of middling size\n\n" + "y" * 150)
    assert len(CalibrationDatasetLoader.v3(cache_dir=str(tmp_path))) == 2 and len(CalibrationDatasetLoader.v3(max_samples=1, cache_dir=str(tmp_path))) == 1
    with pytest.raises(RuntimeError):
        CalibrationDatasetLoader.v3(force_download=True)


def test_activation_functions():
    import metal_marlin_b200 as mm
    g, u = torch.randn(3, 16), torch.randn(3, 16)
    assert torch.allclose(mm.swiglu_fused_metal(g, u), torch.nn.functional.silu(g) * u) and torch.allclose(mm.geglu_fused_metal(g, u), torch.nn.functional.gelu(g) * u)
    assert torch.equal(mm.relu_metal(g), torch.relu(g)) and torch.allclose(mm.silu_metal(g), torch.nn.functional.silu(g)) and torch.allclose(mm.gelu_metal(g), torch.nn.functional.gelu(g))
    with pytest.raises(ValueError):
        mm.swiglu_fused_metal(g, u[:2])


@pytest.mark.gpu
def test_swiglu_fused_kernel_gpu():
    import metal_marlin_b200 as mm
    torch.manual_seed(0)
    g, u = (torch.randn(2, 5, 256, device="cuda", dtype=torch.bfloat16) for _ in range(2))
    ref = torch.nn.functional.silu(g.float()) * u.float()
    assert torch.allclose(mm.swiglu_fused_metal(g, u).float(), ref, atol=3e-2, rtol=2e-2)


# ------------------------------------------------------------------------------------------------ streamer, packings, padding, router
def test_expert_weight_streamer():
    from metal_marlin_b200.memory import ExpertWeightStreamer
    loaded, evicted = [], []
    s = ExpertWeightStreamer(num_experts=16, gpu_cache_size=3, loader=lambda e: loaded.append(e) or {"w": torch.full((2,), float(e))},
                             on_evict=lambda e, o: evicted.append(e))
    for e in (0, 1, 0, 0, 2):
        s.get_expert_weights(e)
    assert list(s.gpu_cache) == [1, 0, 2] and s.hits == 2 and s.misses == 3 and loaded == [0, 1, 2]
    s.get_expert_weights(3)                       # over budget: among the older half {1}, the coldest goes
    assert evicted == [1] and 1 not in s.gpu_cache and s.evictions == 1 and s.access_counts[1] == 0
    assert float(s.get_expert_weights(3)["w"][0]) == 3.0 and s.hit_rate() == pytest.approx(3 / 7)
    for e in (5, 5, 5, 6):                         # each load evicts again; what is not resident and recurs is predicted
        s.get_expert_weights(e)
    pred = s.predicted_experts(4)
    assert all(p not in s.gpu_cache for p in pred) and len(s.gpu_cache) == 3
    assert s.prefetch_experts([9, 99, 9]) == 1 and 9 in s.gpu_cache
    with pytest.raises(ValueError):
        s.get_expert_weights(16)
    plain = ExpertWeightStreamer(4, 2)
    assert plain.get_expert_weights(1) == {"expert_idx": 1, "resident": True}


def test_marlin_gptq_packing_round_trip():
    import metal_marlin_b200 as mm
    from metal_marlin_b200.converters import torch_compat as tc
    rs = np.random.RandomState(0)
    K, N, gs = 64, 24, 32
    codes = rs.randint(0, 16, (K, N)).astype(np.uint8)
    marlin = tc.pack_along_n(codes)
    assert marlin.shape == (K, N // 8) and marlin.dtype == np.uint32 and np.array_equal(tc.unpack_along_n(marlin, N), codes)
    assert int(marlin[3, 1]) == sum(int(codes[3, 8 + i]) << (4 * i) for i in range(8))
    scales = rs.rand(K // gs, N).astype(np.float32)
    sd = mm.export_for_pytorch(marlin, scales, {"in_features": K, "out_features": N, "group_size": gs})
    assert sd["qweight"].shape == (K // 8, N) and sd["qweight"].dtype == np.int32 and np.array_equal(tc.unpack_along_k(sd["qweight"]), codes)
    assert int(sd["qweight"].view(np.uint32)[2, 5]) == sum(int(codes[16 + i, 5]) << (4 * i) for i in range(8))
    assert sd["g_idx"].tolist() == [i // gs for i in range(K)] and sd["bits"].tolist() == [4] and sd["scales"].dtype == np.float16
    back, sc, g = mm.import_from_pytorch(sd)
    assert np.array_equal(back, marlin) and g == gs and np.array_equal(sc, scales.astype(np.float16))
    del sd["group_size"]
    assert mm.import_from_pytorch(sd)[2] == gs                                 # inferred from the shapes
    with pytest.raises(ValueError):
        mm.export_for_pytorch(marlin, scales, {"in_features": K, "out_features": N + 8, "group_size": gs})
    with pytest.raises(ValueError):
        tc.pack_along_n(codes[:, :5])


def test_padding_cholesky_and_aliases():
    import metal_marlin_b200 as mm
    x = torch.arange(15.).reshape(3, 5)
    p, n = mm.pad_to_multiple(x, -1, 4)
    assert p.shape == (3, 8) and n == 3 and torch.equal(p[:, :5], x) and (p[:, 5:] == 0).all() and torch.equal(mm.unpad(p, 1, n), x)
    same, z = mm.pad_to_multiple(x, 0, 3)
    assert same is x and z == 0 and mm.unpad(x, 0, 0) is x
    with pytest.raises(ValueError):
        mm.pad_to_multiple(x, 0, 0)
    rs = np.random.RandomState(0)
    A = rs.randn(12, 6)
    H = A.T @ A
    L = mm.cholesky_decompose(H, 1e-6)
    assert L.dtype == np.float64 and np.allclose(np.tril(L), L) and np.allclose(L @ L.T, H + 1e-6 * np.trace(H) / 6 * np.eye(6), atol=1e-5)
    assert np.isfinite(mm.cholesky_decompose(np.ones((4, 4)), 1e-6)).all()       # singular input: damping takes care of it
    from metal_marlin_b200.trellis import TrellisModelConfig
    assert mm.TrellisConfig is TrellisModelConfig


def test_fast_router_and_hot_pairs():
    from metal_marlin_b200.moe import MoERouterCpp
    torch.manual_seed(0)
    E, H, K = 8, 32, 2
    w = torch.randn(E, H)
    r = MoERouterCpp(E, H, K, max_batch_tokens=64, hot_pair_cache_capacity=2, hot_pair_threshold=3, device="cpu")
    assert (r.num_experts, r.hidden_dim, r.top_k, r.hot_pair_count) == (E, H, K, 0)
    x = torch.randn(10, H)
    out = r.route_batch(x, w.numpy())
    p = torch.softmax(x @ w.t(), -1)
    wt, ids = p.topk(K, -1)
    assert torch.equal(out.expert_ids.long(), ids) and torch.allclose(out.expert_weights, wt / wt.sum(-1, keepdim=True), atol=1e-5)
    assert out.num_tokens == 10 and out.top_k == 2
    bias = torch.zeros(E)
    bias[5] = 50.0
    assert (r.route_batch(x, w, bias.numpy()).expert_ids[:, 0] == 5).all()
    bits = x.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)       # raw bf16 patterns, as the reference passes them
    ob = r.route_batch(bits, w)
    assert torch.equal(ob.expert_ids.long(), torch.softmax(x.to(torch.bfloat16).float() @ w.t(), -1).topk(K, -1).indices)
    with pytest.raises(TypeError):
        r.route_batch(x.numpy(), w)
    with pytest.raises(ValueError):
        r.route_batch(torch.randn(65, H), w)
    with pytest.raises(ValueError):
        MoERouterCpp(4, 8, 5)
    # a token repeated makes its leading pair hot after `threshold` sightings; the cache holds `capacity` pairs
    r.reset_hot_pair_cache()
    one = x[:1].repeat(5, 1)
    o1 = r.route_batch(one, w)
    pair = tuple(sorted(o1.expert_ids[0].tolist()))
    assert o1.hot_pairs == [pair] and o1.hot_pair_hits == 2 and r.hot_pair_count == 1
    for i in (1, 2, 3):
        r.route_batch(x[i:i + 1].repeat(3, 1), w)
    assert r.hot_pair_count <= 2
    r.reset_hot_pair_cache()
    assert r.hot_pair_count == 0


def test_expert_buffer_pool():
    import metal_marlin_b200 as mm
    mm.clear_expert_buffer_pool()
    assert not mm.is_expert_buffer_pool_available() and mm.get_expert_buffer_pool() is None
    with pytest.raises(RuntimeError):
        mm.allocate_expert_weight_buffer(64)
    assert mm.initialize_expert_buffer_pool("cpu", heap_size=1 << 16) and mm.is_expert_buffer_pool_available()
    pool = mm.get_expert_buffer_pool()
    a, b = mm.allocate_expert_weight_buffer(1000), mm.allocate_expert_weight_buffer(3000)
    assert a.dtype == torch.uint8 and a.numel() == 1000 and pool.offset_of(b) >= 1000 and pool.stats()["used"] >= 4000
    pool.free(a)
    c = mm.allocate_expert_weight_buffer(900)
    assert pool.offset_of(c) == 0                                            # best fit reuses the freed block
    assert mm.initialize_expert_buffer_pool("cpu") and mm.get_expert_buffer_pool() is pool      # a second call keeps the pool
    mm.clear_expert_buffer_pool()
    assert not mm.is_expert_buffer_pool_available()


def test_block_sparse_mask_object():
    import metal_marlin_b200 as mm
    from metal_marlin_b200.attention import BlockSparseMask, block_sparse_attention_metal
    m = BlockSparseMask.create_sliding_window(seq_len=1000, window_size=200, block_size=64)
    assert m.num_q_blocks == m.num_k_blocks == 16 and m.mask_bits.shape == (16, 1) and m.mask_bits.dtype == torch.int64
    d = m.dense()
    for i in range(16):
        first = max(0, min((i + 1) * 64, 1000) - 200) // 64
        assert d[i].tolist() == [first <= j <= i for j in range(16)]
    assert m.is_active(5, 5) and m.is_active(5, 2) and not m.is_active(5, 1) and not m.is_active(5, 6) and 0 < m.density < 0.35
    wide = BlockSparseMask.create_sliding_window(seq_len=64 * 130, window_size=64 * 130, block_size=64)      # more than one 64-bit word, bit 63 in use
    assert wide.mask_bits.shape == (130, 3) and wide.is_active(129, 63) and wide.is_active(129, 64) and wide.is_active(129, 129) and not wide.is_active(3, 64)
    assert torch.equal(wide.dense(), torch.tril(torch.ones(130, 130, dtype=torch.bool)))
    bb = BlockSparseMask.create_bigbird(512, num_random_blocks=1, num_global_blocks=1, window_size=128, block_size=64)
    db = bb.dense()
    assert db[:, 0].all() and db[0, :].all() and db.diagonal().all() and db.sum(1).min() >= 3
    assert torch.equal(db, BlockSparseMask.create_bigbird(512, 1, 1, 128, 64).dense())                      # the random blocks are seeded
    lf = BlockSparseMask.create_longformer(512, window_size=128, global_token_indices=(0, 300), block_size=64).dense()
    assert lf[4, :].all() and lf[:, 4].all() and lf[7, 6] and not lf[7, 2]
    el = torch.zeros(100, 150, dtype=torch.bool)
    el[10, 140] = True
    fd = BlockSparseMask.from_dense_mask(el, 32, 64)
    assert (fd.num_q_blocks, fd.num_k_blocks) == (4, 3) and fd.dense().nonzero().tolist() == [[0, 2]]
    add = torch.full((64, 64), float("-inf"))
    add[:, :32] = 0
    assert BlockSparseMask.from_dense_mask(add, 32, 32).dense().tolist() == [[True, False], [True, False]]
    # attention through the mask matches the element-mask oracle
    torch.manual_seed(0)
    S = 256
    q, k, v = (torch.randn(1, 2, S, 32) for _ in range(3))
    sm = BlockSparseMask.create_sliding_window(S, 96, 64)
    out = mm.block_sparse_attention_metal(q, k, v, sm, causal=True)
    ref = torch.nn.functional.scaled_dot_product_attention(q, k, v, attn_mask=sm.element_mask(causal=True))
    assert torch.allclose(out, ref, atol=1e-5)
    rect = BlockSparseMask.from_dense_mask(torch.ones(64, 128, dtype=torch.bool), 32, 64)
    o2 = block_sparse_attention_metal(q[:, :, :64], k[:, :1, :128], v[:, :1, :128], rect)
    r2 = torch.nn.functional.scaled_dot_product_attention(q[:, :, :64], k[:, :1, :128].expand(-1, 2, -1, -1), v[:, :1, :128].expand(-1, 2, -1, -1))
    assert torch.allclose(o2, r2, atol=1e-5)
    with pytest.raises(ValueError):
        block_sparse_attention_metal(q[:, :, :100], k, v, sm)


def test_batch_aware_lora_dispatch():
    """Reference ``tests/test_batch_aware_lora.py``: per-row adapters over a quantized base, ``-1`` = no adapter."""
    from metal_marlin_b200.layers import MMFP4Linear, MixedPrecisionLinear, QuantizedLinear, apply_lora
    torch.manual_seed(0)
    in_f, out_f, rank = 64, 16, 4
    lin = MMFP4Linear.from_float(torch.randn(out_f, in_f), group_size=32, device="cpu")
    x = torch.randn(4, in_f)
    u, v = torch.randn(2, in_f, rank), torch.randn(2, rank, out_f)
    idx = torch.tensor([0, 1, -1, 0])
    base = lin(x).float()
    out = lin.batch_aware_dispatch(x, u, v, idx).float()
    want = base.clone()
    for t, a in enumerate(idx.tolist()):
        if a >= 0:
            want[t] += (x[t] @ u[a]) @ v[a]
    assert torch.allclose(out, want, atol=0.15, rtol=1e-2) and torch.allclose(out[2], base[2])      # bf16 outputs: one rounding of the sum
    assert not torch.allclose(out[0], base[0])
    assert torch.equal(lin.batch_aware_dispatch(x).float(), base)
    # lists of adapters with different ranks, a scaling factor, and one index per sequence of a [batch, seq, in] input
    ul, vl = [torch.randn(in_f, 2), torch.randn(in_f, 6)], [torch.randn(2, out_f), torch.randn(6, out_f)]
    x3 = torch.randn(2, 3, in_f)
    q8 = QuantizedLinear.from_float(torch.randn(out_f, in_f), "int8", 32, device="cpu")
    o3 = q8.batch_aware_dispatch(x3, ul, vl, torch.tensor([1, 0]), scaling=0.5).float()
    w3 = q8(x3).float()
    w3[0] += 0.5 * (x3[0] @ ul[1]) @ vl[1]
    w3[1] += 0.5 * (x3[1] @ ul[0]) @ vl[0]
    assert o3.shape == (2, 3, out_f) and torch.allclose(o3, w3, atol=0.15, rtol=1e-2)
    mp = MixedPrecisionLinear(torch.randn(out_f, 128), "bf16", device="cpu")
    xb = torch.randn(4, 128, dtype=torch.bfloat16)
    ub, vb = torch.randn(2, 128, rank, dtype=torch.bfloat16), torch.randn(2, rank, out_f, dtype=torch.bfloat16)
    ob = mp.batch_aware_dispatch(xb, ub, vb, torch.tensor([0, -1, 1, 0]))
    assert ob.shape == (4, out_f) and torch.allclose(ob[1].float(), mp(xb)[1].float()) and not torch.allclose(ob[2].float(), mp(xb)[2].float())
    acc = torch.zeros(3, out_f)
    apply_lora(acc, torch.ones(3, in_f), u, v, torch.tensor([1, 1, 1]))
    assert torch.allclose(acc[0], torch.ones(in_f) @ u[1] @ v[1], atol=1e-4) and torch.equal(acc[0], acc[2])
    with pytest.raises(ValueError):
        apply_lora(acc, torch.ones(3, in_f), u, v, torch.tensor([0, 2, 0]))
    with pytest.raises(ValueError):
        apply_lora(acc, torch.ones(3, in_f), u, v, torch.tensor([0, 1]))
