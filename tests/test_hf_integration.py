"""HF integration on a tiny Llama built from a config (reference: tests/test_layer_replacement.py,
test_model_utils.py)."""
import pytest
import torch

transformers = pytest.importorskip("transformers")

from metal_marlin_b200.hf import find_linear_layers, find_moe_layers, load_prequantized_mmfp4_model, replace_linear_layers


def _tiny_llama():
    cfg = transformers.LlamaConfig(vocab_size=256, hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                                   num_key_value_heads=2, max_position_embeddings=64)
    torch.manual_seed(0)
    return transformers.LlamaForCausalLM(cfg).eval()


@pytest.mark.parametrize("fmt", ["fp4", "int8"])
def test_replace_linear_layers_keeps_the_model_working(fmt):
    model = _tiny_llama()
    ids = torch.arange(12).view(1, 12)
    with torch.no_grad():
        ref = model(ids).logits
    names = [n for n, _ in find_linear_layers(model)]
    assert "model.layers.0.self_attn.q_proj" in names and not any("lm_head" in n for n in names)
    st = replace_linear_layers(model, fmt=fmt, group_size=64)
    assert st["replaced"] == 14 and st["bytes_after"] < st["bytes_before"] * (0.4 if fmt == "fp4" else 0.6)
    with torch.no_grad():
        got = model(ids).logits
    rel = (got - ref).abs().max() / ref.abs().max()
    assert rel < (0.5 if fmt == "fp4" else 0.1) and (got.argmax(-1) == ref.argmax(-1)).float().mean() > (0.5 if fmt == "fp4" else 0.9)
    assert find_moe_layers(model) == []


def test_load_prequantized_checkpoint_into_meta_model(tmp_path):
    from metal_marlin_b200.formats.safetensors_io import save_file
    from metal_marlin_b200.quant.convert import convert_model
    model = _tiny_llama()
    src = tmp_path / "float"
    src.mkdir()
    save_file({k: v.contiguous() for k, v in model.state_dict().items() if "rotary" not in k}, str(src / "model.safetensors"), metadata={"format": "pt"})
    model.config.save_pretrained(str(src))
    out = tmp_path / "q"
    convert_model(str(src), str(out), "mmfp4", 64)
    with torch.device("meta"):
        shell = transformers.LlamaForCausalLM(model.config)
    st = load_prequantized_mmfp4_model(shell, str(out))
    assert st["quantized"] == 14 and st["dense"] >= 6
    shell.eval()
    ids = torch.arange(12).view(1, 12)
    with torch.no_grad():
        ref, got = model(ids).logits, shell(ids).logits
    assert torch.isfinite(got).all() and (got - ref).abs().max() / ref.abs().max() < 0.5
