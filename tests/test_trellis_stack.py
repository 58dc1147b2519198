"""Trellis container round trip and the trellis causal LM (reference: tests/test_trellis_loader.py,
test_trellis_linear.py, test_trellis_model.py, test_trellis_generate.py)."""
import os

import pytest
import torch

from metal_marlin_b200.formats import trellis as tr
from metal_marlin_b200.formats.safetensors_io import save_file
from metal_marlin_b200.models.config import get_preset
from metal_marlin_b200.quant.convert import random_hf_state
from metal_marlin_b200.trellis import GenerationConfig, TrellisForCausalLM, TrellisGenerator


@pytest.mark.parametrize("bits", [2, 3, 5, 8])
def test_pack_unpack_roundtrip(bits):
    torch.manual_seed(bits)
    codes = torch.randint(0, 1 << bits, (37, 53), dtype=torch.uint8)
    blob = tr.pack_codes(codes, bits)
    assert int(blob[0]) == bits and blob.numel() == 1 + 3 * 4 * tr.tile_bytes(bits)
    back, b = tr.unpack_codes(blob, 37, 53)
    assert b == bits and torch.equal(back, codes)
    with pytest.raises(ValueError):
        tr.unpack_codes(blob.to(torch.int16), 37, 53)


def _float_ckpt(tmp_path, preset):
    cfg = get_preset(preset)
    d = str(tmp_path / "float")
    os.makedirs(d)
    save_file(random_hf_state(cfg, seed=3), os.path.join(d, "model.safetensors"), metadata={"format": "pt"})
    cfg.save_pretrained(d)
    return cfg, d


@pytest.mark.parametrize("container", ["v3", "v2"])
def test_containers_roundtrip(tmp_path, container):
    cfg, d = _float_ckpt(tmp_path, "tiny-llama")
    out = str(tmp_path / "q")
    st = tr.quantize_model_trellis(d, out, bits=4, group_size=64, container=container)
    assert st["quantized"] > 0 and st["mean_rel_rmse"] < 0.15
    ld = tr.TrellisModelLoader(out)
    assert ld.format == ("v3_hf_shards" if container == "v3" else "v2_layers") and ld.bit_histogram() == {4: st["quantized"]}
    name = "model.layers.0.self_attn.q_proj.weight"
    tw = ld.load_weight(name)
    from metal_marlin_b200.formats.safetensors_io import SafetensorsFile
    with SafetensorsFile(os.path.join(d, "model.safetensors")) as sf:
        w = sf.get_tensor(name).float()
    assert (tw.dequantize() - w).abs().max() < 0.1 * w.abs().max() + 1e-3
    assert ld.has_tensor("model.norm.weight")


@pytest.mark.parametrize("preset", ["tiny-llama", "tiny-mla-moe"])
def test_trellis_lm_tracks_float_model(tmp_path, preset):
    cfg, d = _float_ckpt(tmp_path, preset)
    out = str(tmp_path / "q")
    tr.quantize_model_trellis(d, out, bits=8, group_size=64)
    lm = TrellisForCausalLM.from_pretrained(out, device="cpu")
    # float oracle: the same decoder on FP4-from-float weights is too lossy to compare against; use 8-bit trellis
    # vs a second, independent 8-bit load and check determinism + sane logits, then compare against 6-bit
    ids = list(range(3, 19))
    lg = lm.forward_logits(ids)
    assert lg.shape == (16, cfg.vocab_size) and torch.isfinite(lg).all()
    out6 = str(tmp_path / "q6")
    tr.quantize_model_trellis(d, out6, bits=6, group_size=64)
    lg6 = TrellisForCausalLM.from_pretrained(out6, device="cpu").forward_logits(ids)
    # MoE: a near-tie in the router may flip an expert between the two bit widths, so bound the typical error tightly
    # and the worst element loosely
    rel = (lg - lg6).abs() / lg.abs().max()
    assert float(rel.median()) < 0.03 and float(rel.max()) < (0.25 if preset == 'tiny-llama' else 0.7)
    toks = lm.generate([ids], max_new_tokens=5)
    assert len(toks[0]) == 5 and toks == lm.generate([ids], max_new_tokens=5)
    gen = TrellisGenerator(lm)
    greedy = gen.generate(ids, GenerationConfig(max_new_tokens=5, do_sample=False, repetition_penalty=1.0))
    assert greedy == toks[0]
    sampled = list(gen.stream_generate(ids, GenerationConfig(max_new_tokens=4, temperature=0.8, seed=1)))
    assert len(sampled) == 4 and all(0 <= t < cfg.vocab_size for t in sampled)
