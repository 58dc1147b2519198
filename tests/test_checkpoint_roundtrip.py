"""Checkpoint writers and loaders: marlin_fp4 (single file) and mmfp4 (sharded + index) written from a
float HF-named state dict, then loaded unchanged into the engine.  Modelled on the reference's
tests/test_mmfp4_loader.py and tests/test_packed_format.py."""
import json
import os

import pytest
import torch

from metal_marlin_b200.formats import fp4
from metal_marlin_b200.formats.mmfp4_loader import MMFP4ModelLoader, extract_layer_index, name_variants
from metal_marlin_b200.formats.safetensors_io import SafetensorsFile, load_file, save_file
from metal_marlin_b200.models.config import get_preset
from metal_marlin_b200.models.mmfp4_causal_lm import MMFP4ForCausalLM
from metal_marlin_b200.quant.convert import (convert_model, random_hf_state, save_random_checkpoint,
                                             should_quantize_tensor)


def test_safetensors_roundtrip_all_dtypes(tmp_path):
    t = {"a": torch.randn(3, 4), "b": torch.randn(5).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int32),
         "d": torch.randn(2, 2).half(), "e": torch.tensor([1, 2], dtype=torch.uint8)}
    p = str(tmp_path / "x.safetensors")
    save_file(t, p, metadata={"k": "v"}, dtype_overrides={"c": "U32"})
    with SafetensorsFile(p) as f:
        assert f.metadata == {"k": "v"} and f.dtype_str("c") == "U32"
    back = load_file(p)
    for k in t:
        assert torch.equal(back[k], t[k]), k


def test_should_quantize_rule():
    w = torch.zeros(16, 64)
    assert should_quantize_tensor("model.layers.0.self_attn.q_proj.weight", w)
    for n in ("model.embed_tokens.weight", "model.norm.weight", "lm_head.weight", "model.layers.0.mlp.gate.weight",
              "model.layers.0.input_layernorm.weight", "x.bias"):
        assert not should_quantize_tensor(n, w)
    assert not should_quantize_tensor("a.weight", torch.zeros(16, 60))
    assert not should_quantize_tensor("a.weight", torch.zeros(16))


def test_name_variants_and_layer_index():
    assert "model.layers.1.x" in name_variants("model.language_model.layers.1.x")
    assert "model.language_model.layers.1.x" in name_variants("model.layers.1.x")
    assert extract_layer_index("model.layers.12.mlp.up_proj.weight") == 12
    assert extract_layer_index("model.embed_tokens.weight") is None


@pytest.mark.parametrize("fmt", ["marlin_fp4", "mmfp4"])
@pytest.mark.parametrize("preset", ["tiny-llama", "tiny-mla-moe"])
def test_checkpoint_loads_and_matches_direct_quantization(tmp_path, fmt, preset):
    cfg = get_preset(preset)
    out = str(tmp_path / "ckpt")
    info = save_random_checkpoint(cfg, out, fmt=fmt, seed=3)
    assert info["quantized"] > 0 and info["mean_rel_rmse"] < 0.2
    qc = json.load(open(os.path.join(out, "quantization_config.json")))
    assert qc["format"] == ("marlin_fp4" if fmt == "marlin_fp4" else "mmfp4_e2m1_marlin")
    loader = MMFP4ModelLoader(out)
    base = "model.layers.0.self_attn.o_proj"
    assert loader.is_quantized(base) and loader.format == fmt
    packed, scales, layout = loader.get_quantized_weight(base)
    w = random_hf_state(cfg, 3)[base + ".weight"].float()
    codes, sc = fp4.quantize_codes(w, loader.get_group_size(base))
    if layout == "marlin_fp4":
        assert packed.shape == (w.shape[1] // 8, w.shape[0])
        c2, s2 = fp4.unpack_marlin_fp4(packed, scales)
    else:
        assert packed.shape == (w.shape[0], w.shape[1] // 8)
        c2, s2 = fp4.unpack_mmfp4(packed, scales)
    assert torch.equal(c2, codes) and torch.equal(s2, sc)
    if fmt == "mmfp4":
        assert os.path.exists(os.path.join(out, "model.safetensors.index.json"))
        assert len(loader.load_layer(1)) > 0
    lm = MMFP4ForCausalLM.from_pretrained(out, device="cpu")
    toks = lm.generate([[1, 2, 3, 4, 5]], max_new_tokens=4)[0]
    assert len(toks) == 4 and all(0 <= t < cfg.vocab_size for t in toks)


def test_language_model_prefix_alias(tmp_path):
    cfg = get_preset("tiny-llama")
    sd = {("model.language_model." + k[len("model."):] if k.startswith("model.") else k): v
          for k, v in random_hf_state(cfg, 0).items()}
    fdir = tmp_path / "f"
    fdir.mkdir()
    save_file(sd, str(fdir / "model.safetensors"))
    cfg.save_pretrained(str(fdir))
    convert_model(str(fdir), str(tmp_path / "q"), "mmfp4", 128)
    lm = MMFP4ForCausalLM.from_pretrained(str(tmp_path / "q"), device="cpu")
    assert len(lm.generate([[5, 6, 7]], max_new_tokens=2)[0]) == 2


@pytest.mark.parametrize("preset", ["tiny-llama", "tiny-mla-moe"])
def test_rotated_checkpoint_loads_with_its_rotation(tmp_path, preset):
    """A checkpoint whose matrices are stored in the block-Hadamard-rotated basis (``<name>.hadamard_block_size`` beside
    them, as MR-GPTQ writes) must give the logits of the same model stored unrotated, up to 4-bit rounding; ignoring the
    rotation tensors gives unrelated logits."""
    import torch
    from metal_marlin_b200.models.config import get_preset
    from metal_marlin_b200.models.mmfp4_causal_lm import MMFP4ForCausalLM
    from metal_marlin_b200.quant.convert import save_random_checkpoint
    cfg = get_preset(preset)
    plain, rotated = str(tmp_path / "plain"), str(tmp_path / "rot")
    save_random_checkpoint(cfg, plain, seed=5)
    save_random_checkpoint(cfg, rotated, seed=5, hadamard_block=32)
    ids = torch.randint(0, cfg.vocab_size, (24,), generator=torch.Generator().manual_seed(1)).tolist()
    a = MMFP4ForCausalLM.from_pretrained(plain, device="cpu")
    b = MMFP4ForCausalLM.from_pretrained(rotated, device="cpu")
    assert b.model.layers[0].o.hadamard_block == 32 and a.model.layers[0].o.hadamard_block == 0
    la, lb = a.forward_logits(ids), b.forward_logits(ids)
    cos = torch.nn.functional.cosine_similarity(la.flatten(), lb.flatten(), dim=0)
    assert cos > 0.8, cos           # two 4-bit roundings of one random model agree to about 0.9
    # the same rotated bytes read without their rotation: wrong model
    for L in b.model.layers:
        for v in vars(L).values():
            if hasattr(v, "hadamard_block"):
                v.hadamard_block = 0
    lc = b.forward_logits(ids)
    assert torch.nn.functional.cosine_similarity(la.flatten(), lc.flatten(), dim=0) < 0.5
