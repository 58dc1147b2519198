"""EXL3-style checkpoints (format detection, regrouping into the layer-wise layout, conversion to FP4) and the LDLQ quantizer.
Reference: tests/test_exl3_loader.py, tests/test_ldlq.py, tests/test_ldl_decomp.py, tests/test_viterbi_quant.py."""
import json
import os

import pytest
import torch

from metal_marlin_b200.converters import exl3
from metal_marlin_b200.formats import trellis as tr
from metal_marlin_b200.formats.safetensors_io import SafetensorsFile, save_file
from metal_marlin_b200.models.config import get_preset
from metal_marlin_b200.models.mmfp4_causal_lm import MMFP4ForCausalLM
from metal_marlin_b200.quant import ldlq
from metal_marlin_b200.quant.convert import random_hf_state
from metal_marlin_b200.trellis.lm import TrellisForCausalLM


def _trellis_ckpt(tmp_path, bits=6):
    cfg = get_preset("tiny-llama")
    d = str(tmp_path / "float")
    os.makedirs(d)
    save_file(random_hf_state(cfg, seed=3), os.path.join(d, "model.safetensors"), metadata={"format": "pt"})
    cfg.save_pretrained(d)
    out = str(tmp_path / "exl3")
    tr.quantize_model_trellis(d, out, bits=bits, group_size=64, container="v3")
    return cfg, out


def test_detect_formats_and_model_card(tmp_path):
    cfg, ck = _trellis_ckpt(tmp_path)
    info = exl3.detect_exl3_format(ck)
    assert info["format"] in ("single", "sharded") and info["config"]["hidden_size"] == cfg.hidden_size
    lw = str(tmp_path / "lw")
    st = exl3.convert_sharded_to_layerwise(ck, lw)
    assert st["layers"] == cfg.num_hidden_layers and st["matrices"] > 0 and st["base_tensors"] > 0
    info2 = exl3.detect_exl3_format(lw)
    assert info2["format"] == "layerwise" and info2["num_layers"] == cfg.num_hidden_layers
    assert exl3.convert_sharded_to_layerwise(lw, str(tmp_path / "x"))["already_layerwise"]
    with pytest.raises(FileNotFoundError):
        exl3.detect_exl3_format(str(tmp_path))
    assert exl3.parse_layer_index("model.layers.42.mlp.gate_proj.weight") == 42 and exl3.parse_layer_index("lm_head.weight") is None
    card = exl3.parse_model_card("someone/Llama-3.1-8B-Instruct-exl3-4.25bpw")
    assert card == {"base_model": "Llama-3.1-8B-Instruct", "bpw": 4.25, "is_exl3": True}


def test_layerwise_regrouping_loads_the_same_model(tmp_path):
    cfg, ck = _trellis_ckpt(tmp_path)
    ids = list(range(3, 15))
    want = TrellisForCausalLM.from_pretrained(ck, device="cpu").forward_logits(ids)
    # a checkpoint without the index files (tensor names only): shapes and bits are inferred while regrouping
    bare = str(tmp_path / "bare")
    os.makedirs(bare)
    tensors = {}
    for fn in os.listdir(ck):
        if fn.endswith(".safetensors"):
            with SafetensorsFile(os.path.join(ck, fn)) as sf:
                for k in sf.keys():
                    tensors[k] = sf.get_tensor(k)
    save_file(tensors, os.path.join(bare, "model.safetensors"))
    with open(os.path.join(ck, "config.json")) as f, open(os.path.join(bare, "config.json"), "w") as g:
        g.write(f.read())
    assert exl3.detect_exl3_format(bare)["format"] == "single"
    lm = exl3.load_exl3_from_hub(bare, device="cpu")           # a local directory: regrouped next to it, then loaded
    assert os.path.isdir(bare + "-layerwise/layer_0000")
    torch.testing.assert_close(lm.forward_logits(ids), want)


def test_convert_exl3_to_marlin_runs_on_the_fp4_engine(tmp_path):
    cfg, ck = _trellis_ckpt(tmp_path, bits=8)
    out = str(tmp_path / "mmfp4")
    st = exl3.convert_exl3_to_marlin(ck, out, fmt="mmfp4", group_size=64)
    assert st["layers_converted"] > 0 and not st["errors"] and st["total_params"] > 0 and 0 < st["mean_rel_rmse"] < 0.15
    assert st["compression_ratio"] > 1.5                                  # 8-bit codes -> 4-bit codes + group scales
    ids = list(range(3, 15))
    a = TrellisForCausalLM.from_pretrained(ck, device="cpu").forward_logits(ids)
    b = MMFP4ForCausalLM.from_pretrained(out, device="cpu").forward_logits(ids)
    assert torch.nn.functional.cosine_similarity(a.flatten(), b.flatten(), dim=0) > 0.9
    assert exl3.convert_exl3_to_marlin(str(tmp_path / "missing"), out)["errors"]
    tw = tr.quantize_trellis(torch.randn(64, 128) * 0.05, 5, 64)
    packed, sc, err = exl3.exl3_layer_to_marlin(tw, 64)
    assert packed.shape == (128 // 8, 64) and sc.shape == (2, 64) and err < 0.15


def test_block_ldl_factors_the_hessian():
    torch.manual_seed(0)
    X = torch.randn(500, 64)
    H = X.t() @ X
    L, D = ldlq.block_ldl(H, 16, damp=0.0)
    assert D.shape == (4, 16, 16)
    torch.testing.assert_close(ldlq.ldl_reconstruct(L, D), H.double(), rtol=1e-9, atol=1e-7)
    assert float(L.triu(1).abs().max()) < 1e-12 or float(torch.triu(L, 16).abs().max()) == 0.0
    for i in range(4):      # identity blocks on the diagonal
        torch.testing.assert_close(L[16 * i:16 * i + 16, 16 * i:16 * i + 16], torch.eye(16, dtype=torch.float64))
    with pytest.raises(ValueError):
        ldlq.block_ldl(torch.eye(20), 16)


@pytest.mark.parametrize("bits", [2, 3, 4])
def test_ldlq_beats_nearest_rounding_on_the_hessian_metric(bits):
    torch.manual_seed(1)
    n = 256
    X = torch.randn(3000, 32) @ torch.randn(32, n) + 0.3 * torch.randn(3000, n)      # strongly correlated inputs
    H = X.t() @ X
    w = torch.randn(96, n) * 0.05
    a = ldlq.ldlq_quantize(w, H, bits, 128)
    b = ldlq.ldlq_quantize(w, None, bits, 128)
    rtn = ldlq.proxy_error(w, b.dequantized, H)
    assert a.proxy_error < 0.35 * rtn                                                  # error feedback pays on the output metric
    # the container carries exactly what the quantizer decided, and the identity Hessian is plain nearest-grid rounding
    torch.testing.assert_close(a.weight.dequantize(), a.dequantized, rtol=0, atol=1e-6)
    torch.testing.assert_close(b.dequantized, tr.quantize_trellis(w, bits, 128).dequantize(), rtol=0, atol=1e-6)
    assert a.weight.bits == bits
    # the layer output on held-out inputs improves too
    Xt = torch.randn(400, 32) @ torch.randn(32, n) * 0 + X[:400]
    ea = (Xt @ (w - a.dequantized).t()).pow(2).mean()
    eb = (Xt @ (w - b.dequantized).t()).pow(2).mean()
    assert ea < 0.5 * eb


def test_ldlq_rejects_ragged_shapes_and_tile_search_is_nearest():
    with pytest.raises(ValueError):
        ldlq.ldlq_quantize(torch.randn(8, 40), None, 4, 16)
    t = torch.tensor([[0.31, -0.9, 0.02]])
    codes, dq = ldlq.quantize_tile_viterbi(t, torch.tensor(0.1), 4)
    grid = tr.trellis_grid(4) * 0.1
    want = torch.stack([grid[(grid - v).abs().argmin()] for v in t[0]])
    torch.testing.assert_close(dq[0], want.to(dq.dtype))
    assert codes.dtype == torch.uint8


def test_exl3_style_pipeline_hessians_feedback_and_mixed_bits(tmp_path):
    """``quantize --format trellis-v2 --method ldlq --target-bpw``: calibration Hessians per matrix, LDL feedback, bits handed
    out by sensitivity; the container loads and runs, and the average width lands on the target."""
    from metal_marlin_b200.quant.pipeline import quantize_checkpoint
    cfg = get_preset("tiny-llama")
    d = str(tmp_path / "float")
    os.makedirs(d)
    save_file(random_hf_state(cfg, seed=3), os.path.join(d, "model.safetensors"), metadata={"format": "pt"})
    cfg.save_pretrained(d)
    out = str(tmp_path / "q")
    st = quantize_checkpoint(d, out, fmt="trellis-v2", method="ldlq", group_size=64, bits=4, num_samples=4, seq_len=48, device="cpu",
                             target_bpw=3.5)
    assert st["method"] == "ldlq" and st["ldlq"] == st["quantized"] > 0
    assert 3.0 <= st["mean_bpw"] <= 3.5
    ld = tr.TrellisModelLoader(out)
    hist = ld.bit_histogram()
    assert len(hist) >= 2 and min(hist) >= 2 and max(hist) <= 8              # genuinely mixed widths
    lm = TrellisForCausalLM.from_pretrained(out, device="cpu")
    lg = lm.forward_logits(list(range(3, 15)))
    assert torch.isfinite(lg).all()
    with pytest.raises(ValueError):
        quantize_checkpoint(d, str(tmp_path / "bad"), fmt="trellis-v2", method="gptq", device="cpu")
