"""Second-order quantizers (reference: tests/test_gptq*.py, test_mr_gptq.py, test_awq.py, test_hadamard.py,
test_mixed_precision.py)."""
import torch

from metal_marlin_b200.quant import awq, gptq, hadamard, mixed_precision
from metal_marlin_b200.quant.calibration import HessianCollector, load_calibration_tokens
from metal_marlin_b200.quant.rtn import quantize as rtn


def _layer(seed=0, out_f=48, in_f=256, n=512):
    g = torch.Generator().manual_seed(seed)
    W = torch.randn(out_f, in_f, generator=g) * 0.05
    mix = torch.randn(in_f, in_f, generator=g) * 0.3 + torch.eye(in_f)
    X = torch.randn(n, in_f, generator=g) @ mix               # correlated inputs: where GPTQ beats RTN
    return W, X


def test_hadamard_is_orthonormal_involution():
    H = hadamard.hadamard_matrix(64)
    torch.testing.assert_close(H @ H.t(), torch.eye(64), atol=1e-6, rtol=0)
    x = torch.randn(3, 256)
    y = hadamard.block_hadamard(x, 64)
    torch.testing.assert_close(y.view(3, 4, 64), x.view(3, 4, 64) @ H, atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(hadamard.block_hadamard(y, 64), x, atol=1e-5, rtol=1e-5)
    W = torch.randn(8, 256)
    torch.testing.assert_close(hadamard.rotate_weight(W, 128) @ hadamard.block_hadamard(x, 128).t(), W @ x.t(), atol=1e-4, rtol=1e-4)
    spiky = torch.randn(16, 512)
    spiky[:, ::64] *= 20
    assert float(hadamard.kurtosis(spiky).mean()) > 5 > float(hadamard.kurtosis(hadamard.rotate_weight(spiky, 128)).mean())


def test_gptq_beats_rtn_on_output_error_and_stays_on_grid():
    W, X = _layer()
    H = X.t() @ X / X.shape[0]
    ref = X @ W.t()
    for fmt in ("fp4", "int4"):
        for act_order in (False, True):
            cfg = gptq.GPTQConfig(fmt=fmt, group_size=64, act_order=act_order)
            wq, scales, st = gptq.gptq_quantize(W, H, cfg)
            e_gptq = float((X @ wq.t() - ref).pow(2).mean())
            e_rtn = float((X @ rtn(W, fmt, 64).dequantize().t() - ref).pow(2).mean())
            assert e_gptq < 0.8 * e_rtn, (fmt, act_order, e_gptq, e_rtn)
            qt = gptq.to_quantized_tensor(wq, scales, fmt, 64)
            torch.testing.assert_close(qt.dequantize(), wq, atol=1e-5, rtol=1e-3)


def test_mr_gptq_rotation_gate_and_equivalence():
    W, X = _layer(1)
    W[:, 7] *= 25                                             # an outlier channel -> high kurtosis -> rotate
    H = X.t() @ X / X.shape[0]
    cfg = gptq.MRGPTQConfig(fmt="fp4", group_size=128, hadamard_block=128)
    wq, scales, st = gptq.mr_gptq_quantize(W, H, cfg)
    assert st["rotated"] and st["hadamard_block"] == 128
    y = hadamard.block_hadamard(X, 128) @ wq.t()              # runtime: rotate the input, multiply the rotated weight
    e_rot = float((y - X @ W.t()).pow(2).mean())
    wq_plain, _, st2 = gptq.mr_gptq_quantize(W, H, gptq.MRGPTQConfig(fmt="fp4", force_rotation=False))
    e_plain = float((X @ wq_plain.t() - X @ W.t()).pow(2).mean())
    assert not st2["rotated"] and e_rot < e_plain
    smooth = torch.randn(8, 256) * 0.02
    assert not gptq.mr_gptq_quantize(smooth, None, cfg)[2]["rotated"]
    wqs, ss, stats = gptq.quantize_stacked_experts(torch.stack([W, smooth.repeat(6, 1)]), [H, None], cfg)
    assert wqs.shape == (2, 48, 256) and stats[0]["rotated"] and not stats[1]["rotated"]


def test_awq_improves_on_rtn_with_salient_channels():
    W, X = _layer(2)
    X[:, :8] *= 30                                            # salient input channels
    q, s, st = awq.awq_quantize(W, X, "int4", 64)
    assert st["mse"] <= st["mse_rtn"] and s.shape == (256,)
    y = (X / s) @ q.dequantize().t()
    assert float((y - X @ W.t()).pow(2).mean()) <= st["mse_rtn"] * 1.001


def test_hessian_collector_calibration_and_resume(tmp_path):
    c = HessianCollector()
    x = torch.randn(4, 10, 16)
    c.add("l0.q", x[:2]), c.add("l0.q", x[2:])
    torch.testing.assert_close(c.get("l0.q", normalize=False), x.view(-1, 16).t() @ x.view(-1, 16), atol=1e-4, rtol=1e-4)
    c.add_expert("l0.mlp", x.view(-1, 16), torch.tensor([[0, 1]] * 20 + [[2, 1]] * 20), 4)
    assert c.n["l0.mlp.experts.1"] == 40 and c.n["l0.mlp.experts.0"] == 20
    c.save(str(tmp_path / "h.pt"))
    assert HessianCollector.load(str(tmp_path / "h.pt")).names() == c.names()
    toks = load_calibration_tokens("wikitext2", vocab_size=100, num_samples=4, seq_len=32)
    assert len(toks) == 4 and all(len(t) == 32 and max(t) < 100 for t in toks)
    st = gptq.ResumableState(str(tmp_path))
    st.mark("a.weight", {"sq_err": 1.0})
    assert gptq.ResumableState(str(tmp_path)).is_done("a.weight")


def test_mixed_precision_presets_and_bit_allocation():
    p = mixed_precision.policy_for
    assert p("model.layers.3.mlp.experts.7.up_proj.weight", "moe") == mixed_precision.TensorPolicy("fp4", 128)
    assert p("model.layers.3.mlp.shared_experts.up_proj.weight", "moe").group_size == 64
    assert p("model.layers.3.mlp.gate.weight", "moe").fmt == "keep" and p("model.norm.weight", "dense").fmt == "keep"
    assert p("model.layers.0.self_attn.q_proj.weight", "quality").fmt == "int8"
    assert p("model.mtp.0.eh_proj.weight", "moe-mtp").fmt == "int8"
    sens = {"a": {2: 10.0, 4: 1.0, 8: 0.1}, "b": {2: 1.0, 4: 0.5, 8: 0.4}}
    alloc = mixed_precision.allocate_bits(sens, {"a": 100, "b": 100}, target_bpw=4.0, choices=(2, 4, 8))
    assert alloc == {"a": 4, "b": 4} or alloc == {"a": 4, "b": 2}
    assert mixed_precision.allocate_bits(sens, {"a": 100, "b": 100}, target_bpw=3.0, choices=(2, 4, 8)) == {"a": 4, "b": 2}


def test_awq_plan_folds_the_scale_into_the_norm_and_keeps_the_function():
    """Whole-checkpoint AWQ on one synthetic layer: projections behind a norm share a scale vector; after applying the plan the
    float function is unchanged (norm / s, weights * s, router compensated) and the quantized layer output is closer to the
    float one than round-to-nearest when a few input channels dominate."""
    torch.manual_seed(0)
    H, I, E = 128, 192, 4
    p = "model.layers.0."
    sd = {p + "input_layernorm.weight": 1 + 0.1 * torch.randn(H), p + "post_attention_layernorm.weight": 1 + 0.1 * torch.randn(H),
          p + "self_attn.q_proj.weight": torch.randn(H, H) * 0.05, p + "self_attn.k_proj.weight": torch.randn(64, H) * 0.05,
          p + "self_attn.v_proj.weight": torch.randn(64, H) * 0.05, p + "self_attn.o_proj.weight": torch.randn(H, H) * 0.05,
          p + "mlp.gate.weight": torch.randn(E, H) * 0.05, "model.norm.weight": torch.ones(H)}
    for e in range(E):
        sd[p + f"mlp.experts.{e}.gate_proj.weight"] = torch.randn(I, H) * 0.05
        sd[p + f"mlp.experts.{e}.up_proj.weight"] = torch.randn(I, H) * 0.05
        sd[p + f"mlp.experts.{e}.down_proj.weight"] = torch.randn(H, I) * 0.05
    X = torch.randn(400, H)
    X[:, :6] *= 12.0                                     # salient channels
    inputs = {n: X for n in sd if n.endswith(("q_proj.weight", "k_proj.weight", "v_proj.weight", "gate_proj.weight", "up_proj.weight"))}
    plan = awq.awq_plan(sd.keys(), lambda n: sd[n], lambda n: inputs.get(n), "int4", 64, n_grid=10)
    assert set(plan) == {p + "input_layernorm.weight", p + "post_attention_layernorm.weight"}
    g = plan[p + "post_attention_layernorm.weight"]
    assert len(g["consumers"]) == 2 * E and g["compensate"] == [p + "mlp.gate.weight"] and g["alpha"] > 0 and g["mse"] < 0.7 * g["mse_rtn"]
    new = dict(awq.apply_awq_plan(sd.items(), plan))
    assert set(new) == set(sd) and torch.equal(new[p + "self_attn.o_proj.weight"], sd[p + "self_attn.o_proj.weight"])

    def rms(x, w):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * w
    x = torch.randn(8, H)
    for norm, mats in ((p + "input_layernorm.weight", [p + "self_attn.q_proj.weight", p + "self_attn.v_proj.weight"]),
                       (p + "post_attention_layernorm.weight", [p + "mlp.gate.weight", p + "mlp.experts.2.up_proj.weight"])):
        for m in mats:
            torch.testing.assert_close(rms(x, new[norm]) @ new[m].t(), rms(x, sd[norm]) @ sd[m].t(), rtol=1e-4, atol=1e-4)
    # quantized: the scaled weights reproduce the float projection better on the salient data
    from metal_marlin_b200.quant.rtn import quantize
    n, m = p + "post_attention_layernorm.weight", p + "mlp.experts.1.gate_proj.weight"
    ref = X @ sd[m].t()
    e_rtn = ((X @ quantize(sd[m], "int4", 64).dequantize(torch.float32).t()) - ref).pow(2).mean()
    s = plan[n]["scale"]
    e_awq = (((X / s) @ quantize(new[m], "int4", 64).dequantize(torch.float32).t()) - ref).pow(2).mean()
    assert e_awq < 0.8 * e_rtn
