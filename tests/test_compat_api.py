"""The reference facade's names on this engine (``compat_api.py``): packers in the marlin ``[K, N]`` orientation, FP8 tables
and KV helpers, Hadamard rotation with metadata, MoE dispatch bookkeeping, GEMM / attention entry points, RoPE helpers,
precision configuration and allocation, ONNX / vision helpers, memory and dispatch objects, module-level generation.
Parity: reference ``tests/test_quantize.py``, ``test_fp8_utils.py``, ``test_hadamard.py``, ``test_moe_dispatch.py``,
``test_attention.py``, ``test_rope.py`` (the same functions through the package facade)."""
import numpy as np
import pytest
import torch

import metal_marlin_b200 as mm
from metal_marlin_b200 import compat_api as ca


REFERENCE_EXPORTS = (
    "AWQResult AdaptiveQuantResult AdaptiveQuantizer AsyncPipelineScheduler AsyncTransferHandle AsyncTransferManager "
    "BatchDispatchContext CacheConfig CacheConfigTorch CppDispatchInfo ExpertManagerCpp FP4GPTQQuantizer FP4Metal "
    "FP8_E4M3_MAX FP8_E4M3_VALUES FP8_E5M2_MAX FP8_E5M2_VALUES FastInferenceContext GPTQMetal GPTQQuantizer GenerationConfig "
    "HAS_MPS HAS_PYOBJC_METAL HAS_TORCH HadamardMetadata HadamardMetal HeapAllocation HeapAllocatorMetrics HeapBufferPool "
    "HessianCollector HessianManager InferenceRequest InternVLProjector KVCache KVCacheTorch LLaVAProjector LayerBudget "
    "LayerPrecisionSelector LayerQuantConfig LayerSensitivity MLAAttentionCpp MLAKVCache MRGPTQQuantizer MarlinAttention "
    "MarlinLinear MetalHeapAllocator MetalQuantizedLinear MetalQuantizedMoE MetalSampler MixedPrecisionConfig MoEDispatchInfo "
    "MoEPrecisionConfig ModelBudgetAllocation ONNXGraphInfo ONNXOp PipelineScheduler PipelinedLayerDispatcher Precision "
    "QuantizationFormat QuantizationReport Qwen2VLProjector RequestState RoPE SamplingConfig VisionProjector VisionProjectorConfig "
    "YaRNConfig YaRNRoPE apply_hadamard_rotation awq_dequantize awq_quantize awq_quantize_model compute_activation_stats "
    "compute_expert_load compute_fp8_e4m3_values compute_fp8_e5m2_values compute_hessian_metal compute_load_balancing_loss "
    "compute_moe_expert_sensitivity compute_salient_scaling compute_yarn_cos_sin_cache compute_yarn_inv_freq create_causal_mask "
    "create_expert_manager create_rope_from_config create_sliding_window_mask dequant_fp8_e4m3 dequant_fp8_e5m2 "
    "dequantize_fp4_metal dequantize_fp8_e4m3 dequantize_fp8_e5m2 dequantize_kv_cache_fp8 dequantize_kv_cache_fp8_e5m2 "
    "dequantize_mmfp4 detect_architecture detect_projector_type dispatch_batched_gemm_variable_seq dispatch_grouped_attention_variable_seq "
    "expert_gather expert_manager_available expert_scatter_add extract_onnx_weights fast_dispatch_available find_linear_layers "
    "find_moe_layers find_salient_weights flash_attention_metal fused_moe_forward gather_for_experts generate generate_batch "
    "generate_pipelined generate_stream get_fast_context get_onnx_config get_parent_module get_yarn_mscale group_tokens_by_expert "
    "group_tokens_by_expert_full hadamard_matrix hadamard_transform_metal inverse_hadamard_rotation list_onnx_tensors "
    "marlin_gemm_fp4 marlin_gemm_int4 mla_cpp_available mmfp4_fused_qkv mmfp4_gemm normalize_onnx_name pack_fp4_weights "
    "pack_fp4_weights_cpu pack_fp8_weights pack_int4_weights pack_nf4_weights parse_onnx_graph parse_onnx_graph_full "
    "quantize_fp4_metal quantize_kv_cache_fp8 quantize_kv_cache_fp8_e5m2 quantize_linear_layer quantize_moe_experts "
    "quantize_to_fp8 quantize_to_fp8_e4m3 quantize_to_fp8_e5m2 quantize_to_int4 quantize_to_nf4 replace_linear_layers "
    "replace_moe_layers sample_next_token scaled_dot_product_attention_metal scatter_expert_outputs sliding_window_attention_metal "
    "summarize_graph unpack_fp4_weights"
).split()


def test_every_reference_export_resolves():
    """The public names of the reference package (its ``__all__``) all exist here."""
    assert len(REFERENCE_EXPORTS) == 154
    for n in REFERENCE_EXPORTS:
        assert getattr(mm, n) is not None or n.startswith("HAS_"), n
    assert mm.HAS_MPS is False and mm.MarlinLinear is mm.MMFP4Linear


@pytest.mark.parametrize("backend", ["numpy", "torch"])
def test_pack_unpack_round_trips(backend):
    torch.manual_seed(0)
    w = torch.randn(200, 48) * 0.1                      # K = 200 is padded to 256
    packed, scales, meta = ca.pack_fp4_weights(w, 128, output_backend=backend)
    assert tuple(packed.shape) == (32, 48) and tuple(scales.shape) == (2, 48) and meta["orig_K"] == 200 and meta["padded_K"] == 256
    assert (packed.dtype == np.uint32) if backend == "numpy" else (packed.dtype == torch.int32)
    back = torch.as_tensor(np.asarray(ca.unpack_fp4_weights(packed, scales, meta, output_backend=backend), dtype=np.float32)
                           if backend == "numpy" else ca.unpack_fp4_weights(packed, scales, meta, output_backend=backend).float())
    assert back.shape == (200, 48) and float((back - w).abs().max()) < 0.26 * float(w.abs().max())
    with pytest.raises(ValueError):
        ca.pack_fp4_weights(w, 128, pad_k=False)
    # the marlin layout feeds the GEMM entry point
    A = torch.randn(5, 256)
    p2, s2, m2 = ca.pack_fp4_weights(torch.randn(256, 64) * 0.1, 128, output_backend="torch")
    y = ca.marlin_gemm_fp4(A, p2, s2, 128).float()
    ref = A.bfloat16().float() @ ca.unpack_fp4_weights(p2, s2, m2, output_backend="torch").float()
    assert float((y - ref).abs().max()) < 0.05 * float(ref.abs().max()) + 1e-2
    # INT4 with zero points, NF4, FP8
    pi, si, mi = ca.pack_int4_weights(w, 64, output_backend="torch")
    assert tuple(pi.shape) == (25 + 7, 48)[:0] or pi.shape[1] == 48 and "zeros" in mi
    pn, sn, mn = ca.pack_nf4_weights(w[:192], 64, output_backend="torch")
    assert pn.shape == (24, 48) and mn["format"] == "nf4"
    p8, s8, m8 = ca.pack_fp8_weights(w[:128], 64, output_backend="torch")
    d8 = ca.dequant_fp8_e4m3(p8, s8, m8, output_backend="torch").float()
    assert float((d8 - w[:128]).abs().max()) < 0.07 * float(w.abs().max())


def test_fp8_tables_and_kv_helpers():
    v = ca.compute_fp8_e4m3_values()
    assert v.shape == (256,) and float(np.abs(v).max()) == ca.FP8_E4M3_MAX == 448.0 and float(np.abs(ca.FP8_E5M2_VALUES).max()) == 57344.0
    k, vv = torch.randn(2, 4, 10, 64), torch.randn(2, 4, 10, 64)
    for method in ("tensor", "channel", "group"):
        (kc, ks), (vc, vs) = ca.quantize_kv_cache_fp8(k, vv, scale_method=method, group_size=32)
        assert kc.dtype == torch.uint8 and kc.shape == k.shape
        kb, vb = ca.dequantize_kv_cache_fp8(kc, ks, vc, vs, output_dtype=torch.float32)
        assert float((kb - k).abs().max()) < 0.08 * float(k.abs().max())
    (kc, ks), _ = ca.quantize_kv_cache_fp8_e5m2(k, vv)
    assert float((ca.dequantize_fp8_e5m2(kc, ks, torch.float32) - k).abs().max()) < 0.15 * float(k.abs().max())
    codes, scales = ca.quantize_fp4_metal(torch.randn(8, 128), 64)
    assert codes.shape == (8, 128) and ca.dequantize_fp4_metal(codes, scales, 64).shape == (8, 128)


def test_hadamard_rotation_with_metadata():
    w = np.random.RandomState(0).randn(100, 24).astype(np.float32)
    rot, meta = ca.apply_hadamard_rotation(w, block_size=64, axis=0)
    assert rot.shape == (128, 24) and meta.orig_shape == (100, 24) and isinstance(rot, np.ndarray)
    back = ca.inverse_hadamard_rotation(rot, meta)
    assert back.shape == (100, 24) and float(np.abs(back - w).max()) < 1e-4
    x = torch.randn(3, 128)
    y = ca.hadamard_transform_metal(x, 64)
    assert torch.allclose(ca.hadamard_transform_metal(y, 64), x, atol=1e-4)
    assert torch.allclose(y.pow(2).sum(), x.pow(2).sum(), rtol=1e-4)


def test_moe_dispatch_bookkeeping():
    torch.manual_seed(1)
    T, k, E, H = 9, 2, 4, 8
    ids = torch.stack([torch.randperm(E)[:k] for _ in range(T)])
    order, offsets, inverse = ca.group_tokens_by_expert(ids, E)
    flat = ids.reshape(-1)
    assert torch.equal(flat[order], flat[order].sort().values) and int(offsets[-1]) == T * k
    assert torch.equal(order[inverse], torch.arange(T * k))
    info = ca.group_tokens_by_expert_full(ids, E)
    x = torch.randn(T, H)
    g = ca.gather_for_experts(x, info)
    assert g.shape == (T * k, H) and torch.equal(g[0], x[info.sorted_token_indices[0]])
    probs = torch.rand(T, k)
    out = ca.scatter_expert_outputs(g, probs, info)
    assert torch.allclose(out, x * probs.sum(1, keepdim=True), atol=1e-5)
    assert torch.equal(ca.compute_expert_load(ids, E), torch.bincount(flat, minlength=E))
    w = torch.randn(E, H)
    assert ca.expert_gather(w, ids).shape == (T, k, H)
    assert torch.allclose(ca.expert_scatter_add(torch.ones(T, k, H), ids, probs), probs.sum(1, keepdim=True).expand(T, H))
    assert float(ca.compute_load_balancing_loss(torch.softmax(torch.randn(T, E), -1), ids, E)) > 0
    mgr = ca.create_expert_manager(E, k)
    assert ca.expert_manager_available() and mgr.group(ids).num_tokens == T and mgr.load_imbalance(ids) >= 1.0
    d = ca.CppDispatchInfo.build(ids.to(torch.int32), E, token_tile=4)
    assert int(d.num_tiles) >= E - 1 and torch.equal(d.order.long()[d.inverse.long()], torch.arange(T * k))


def test_attention_entry_points_and_masks():
    torch.manual_seed(2)
    B, Hq, Hk, T, D = 1, 4, 2, 12, 32
    q, k, v = torch.randn(B, Hq, T, D), torch.randn(B, Hk, T, D), torch.randn(B, Hk, T, D)
    ref = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
    assert float((ca.flash_attention_metal(q, k, v) - ref).abs().max()) < 3e-2
    assert float((ca.scaled_dot_product_attention_metal(q, k, v, is_causal=True) - ref).abs().max()) < 3e-2
    m = ca.create_sliding_window_mask(T, 4)
    refw = torch.nn.functional.scaled_dot_product_attention(q, k, v, attn_mask=m, enable_gqa=True)
    assert float((ca.sliding_window_attention_metal(q, k, v, 4) - refw).abs().max()) < 3e-2
    assert float((ca.scaled_dot_product_attention_metal(q, k, v, attn_mask=m) - refw).abs().max()) < 1e-5
    cm = ca.create_causal_mask(3, 5)
    assert cm.shape == (1, 1, 3, 5) and cm[0, 0, 0].tolist() == [0, 0, 0, float("-inf"), float("-inf")] and ca.create_causal_mask(1, 7) is None
    lens = torch.tensor([5, 7])
    Q, K = torch.randn(12, Hq, D).bfloat16(), torch.randn(12, Hk, D).bfloat16()
    o = ca.dispatch_grouped_attention_variable_seq(None, Q, K, None, lens, 7, V=K)
    assert o.shape == (12, Hq, D)


def test_rope_helpers():
    from metal_marlin_b200.rope import YaRNConfig
    cfg = YaRNConfig(original_max_position=4096, scale_factor=4.0, rope_theta=10000.0)
    inv = ca.compute_yarn_inv_freq(64, 10000.0, cfg)
    cos, sin = ca.compute_yarn_cos_sin_cache(64, 128, 10000.0, cfg)
    assert inv.shape == (32,) and cos.shape == (128, 32) and ca.get_yarn_mscale(4.0) == pytest.approx(0.1 * np.log(4.0) + 1.0)
    assert ca.get_yarn_mscale(1.0) == 1.0
    rope = ca.RoPE(64)
    x = torch.randn(2, 5, 3, 64)
    pos = torch.arange(5).expand(2, 5)
    y = rope(x, pos)
    assert y.shape == x.shape and torch.allclose(y[:, 0], x[:, 0], atol=1e-6) and torch.allclose(y.norm(dim=-1), x.norm(dim=-1), atol=1e-4)
    hf = {"hidden_size": 256, "num_attention_heads": 4, "rope_theta": 10000.0, "max_position_embeddings": 16384,
          "rope_scaling": {"type": "yarn", "factor": 4.0, "original_max_position_embeddings": 4096}}
    yr = ca.create_rope_from_config(hf)
    assert isinstance(yr, ca.YaRNRoPE) and yr(x, pos).shape == x.shape and ca.create_rope_from_config({"hidden_size": 8, "num_attention_heads": 1}) is None


def test_precision_configuration_and_allocation():
    mp = ca.MixedPrecisionConfig.from_preset("quality")
    assert mp.attention is ca.Precision.INT8 and mp.moe.experts is ca.Precision.FP4 and ca.Precision.INT3.bits == 3
    sel = ca.LayerPrecisionSelector(mp)
    assert sel.select("model.layers.0.input_layernorm.weight").precision is ca.Precision.BF16
    assert not sel.select("model.embed_tokens.weight").quantized and sel.select("model.layers.3.mlp.experts.5.up_proj.weight").quantized
    sens = [ca.LayerSensitivity("a", 1000, {2: 9.0, 4: 1.0, 8: 0.1}), ca.LayerSensitivity("b", 1000, {2: 1.0, 4: 0.5, 8: 0.4})]
    res = ca.AdaptiveQuantizer(target_bpw=5.0, bit_choices=(2, 4, 8)).allocate(sens)
    alloc = res.allocation
    assert alloc.bits_for("a") >= alloc.bits_for("b") and alloc.mean_bpw <= 5.0 + 1e-6 and alloc.total_bytes > 0
    rep = ca.QuantizationReport()
    rep.add("a", "fp4", 4, 0.05, 1000)
    rep.add("b", "int8", 8, 0.01, 3000)
    assert rep.summary()["mean_bpw"] == 7.0 and rep.summary()["worst"] == "a" and "entries" in rep.to_json()
    st = ca.compute_activation_stats(np.random.RandomState(0).randn(4, 6, 16), "rms")
    mask, idx = ca.find_salient_weights(np.zeros((16, 8)), st, 0.25)
    assert st.shape == (16,) and mask.sum() == 4 and len(idx) == 4
    sc = ca.compute_salient_scaling(np.random.RandomState(1).randn(16, 8), mask, None, 8)
    assert sc.shape == (16,) and (sc[~mask] == 1).all() and (sc[mask] >= 1).all()
    H = ca.compute_hessian_metal(torch.randn(50, 16))
    assert H.shape == (16, 16) and torch.allclose(H, H.t())
    s = ca.compute_moe_expert_sensitivity([np.eye(4) * (i + 1) for i in range(3)])
    assert s.shape == (3,) and s[2] > s[0] and abs(s.mean() - 1) < 1e-9
    wq, scales, stats = ca.FP4GPTQQuantizer(group_size=16).quantize_weight(torch.randn(8, 32) * 0.1, H.new_tensor(np.eye(32)))
    assert wq.shape == (8, 32) and scales.shape == (8, 2)


def test_module_helpers_onnx_vision_and_generation(tmp_path):
    import torch.nn as nn
    lin = nn.Linear(128, 64, bias=False)
    qm = ca.quantize_linear_layer(lin, 4, 64, "fp4")
    x = torch.randn(3, 128)
    assert float((qm(x) - lin(x)).detach().abs().max()) < 0.3 * float(lin(x).detach().abs().max())
    model = nn.Sequential(nn.Sequential(nn.Linear(4, 4)))
    parent, attr = ca.get_parent_module(model, "0.0")
    assert parent is model[0] and attr == "0"
    from metal_marlin_b200.converters.onnx import export_linear_stack
    path = str(tmp_path / "m.onnx")
    open(path, "wb").write(export_linear_stack([torch.randn(32, 16), torch.randn(8, 32)]))
    info = ca.parse_onnx_graph_full(path)
    assert info.op_counts and len(info.initializers) >= 2
    assert {t["name"] for t in ca.list_onnx_tensors(path)} == set(info.initializers)
    got = list(ca.extract_onnx_weights(path))
    assert len(got) >= 2 and all(isinstance(a, np.ndarray) for _n, a, _m in got)
    assert ca.normalize_onnx_name("/model/layers.0/self_attn/q_proj/MatMul") == "model.layers.0.self_attn.q_proj.weight"
    assert ca.normalize_onnx_name("onnx::MatMul_12", {"onnx::MatMul_12": ["/model/layers.1/mlp/up_proj/MatMul"]}) == "model.layers.1.mlp.up_proj.weight"
    assert ca.detect_projector_type({"model_type": "qwen2_vl"}) == "qwen2_vl" and ca.detect_projector_type({"model_type": "llava"}) == "llava"
    proj = ca.VisionProjector.build(ca.VisionProjectorConfig("llava", 16, 32), {"w1": torch.randn(32, 16), "w2": torch.randn(32, 32)})
    assert proj(torch.randn(1, 5, 16)).shape == (1, 5, 32)
    from metal_marlin_b200.models.mmfp4_causal_lm import MMFP4ForCausalLM
    lm = MMFP4ForCausalLM.from_config("tiny-llama", device="cpu", seed=0)

    class Cfg:
        max_new_tokens = 4
    want = lm.generate([[1, 2, 3, 4, 5]], max_new_tokens=4)[0]
    assert ca.generate(lm, torch.tensor([1, 2, 3, 4, 5]), Cfg()) == list(want)
    assert ca.generate_batch(lm, torch.tensor([[1, 2, 3, 4, 5]]), Cfg()) == [list(want)]
    h = ca.AsyncTransferManager("cpu").submit({"a": torch.ones(3)})
    assert h.done() and h.wait()["a"].sum() == 3
    ran = []
    with ca.BatchDispatchContext("cpu") as b:
        b.run(lambda: ran.append(1))
    assert ran == [1] and ca.get_fast_context() is ca.get_fast_context() and ca.fast_dispatch_available() in (True, False)
    out = ca.PipelinedLayerDispatcher("cpu").run([{"w": torch.full((2, 2), float(i))} for i in range(3)], lambda i, w, x: x + w["w"].sum(), 0.0)
    assert float(out) == 0 + 4 + 8
