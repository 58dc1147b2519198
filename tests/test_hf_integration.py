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


def _tiny_qwen3_moe():
    cfg = transformers.Qwen3MoeConfig(vocab_size=256, hidden_size=128, intermediate_size=256, moe_intermediate_size=64, num_hidden_layers=2,
                                      num_attention_heads=4, num_key_value_heads=2, head_dim=32, num_experts=8, num_experts_per_tok=2,
                                      max_position_embeddings=64, decoder_sparse_step=1, mlp_only_layers=[], norm_topk_prob=True)
    torch.manual_seed(0)
    return transformers.Qwen3MoeForCausalLM(cfg).eval()


def test_replace_moe_layers_swaps_fused_expert_tensors_for_fp4_banks():
    from metal_marlin_b200.hf import QuantizedMoEExperts, replace_moe_layers_streaming
    model = _tiny_qwen3_moe()
    ids = torch.arange(10).view(1, 10)
    with torch.no_grad():
        ref = model(ids).logits
    assert [n for n, _ in find_moe_layers(model)] == ["model.layers.0.mlp", "model.layers.1.mlp"]
    seen = []
    st = replace_moe_layers_streaming(model, group_size=64, on_layer_complete=lambda name, i, n: seen.append((name, i, n)))
    assert st["replaced"] == 2 and st["experts"] == 16 and st["bytes_after"] < 0.4 * st["bytes_before"]
    assert seen == [("model.layers.0.mlp", 0, 2), ("model.layers.1.mlp", 1, 2)]
    assert isinstance(model.model.layers[0].mlp.experts, QuantizedMoEExperts)
    with torch.no_grad():
        got = model(ids).logits
    cos = torch.nn.functional.cosine_similarity(got.flatten(), ref.flatten(), dim=0)
    assert cos > 0.98 and torch.isfinite(got).all()


def test_module_list_experts_become_a_quantized_block():
    import torch.nn as nn
    from metal_marlin_b200.hf import QuantizedMoEBlock, replace_moe_layers

    class Expert(nn.Module):
        def __init__(self, h, i):
            super().__init__()
            self.gate_proj, self.up_proj, self.down_proj = nn.Linear(h, i, bias=False), nn.Linear(h, i, bias=False), nn.Linear(i, h, bias=False)

        def forward(self, x):
            return self.down_proj(torch.nn.functional.silu(self.gate_proj(x)) * self.up_proj(x))

    class Block(nn.Module):
        def __init__(self, h=128, i=64, e=4, k=2):
            super().__init__()
            self.gate = nn.Linear(h, e, bias=False)
            self.experts = nn.ModuleList([Expert(h, i) for _ in range(e)])
            self.top_k, self.norm_topk_prob = k, True

        def forward(self, x):
            p = torch.softmax(self.gate(x).float(), -1)
            w, idx = torch.topk(p, self.top_k, -1)
            w = w / w.sum(-1, keepdim=True)
            out = torch.zeros_like(x)
            for t in range(x.shape[0]):
                for s in range(self.top_k):
                    out[t] += w[t, s] * self.experts[int(idx[t, s])](x[t])
            return out

    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.mlp = Block()

        def forward(self, x):
            return self.mlp(x)

    torch.manual_seed(1)
    net = Net().eval()
    x = torch.randn(6, 128)
    with torch.no_grad():
        ref = net(x)
    st = replace_moe_layers(net, group_size=64)
    assert st["replaced"] == 1 and isinstance(net.mlp, QuantizedMoEBlock)
    with torch.no_grad():
        got = net(x)
    assert torch.nn.functional.cosine_similarity(got.flatten(), ref.flatten(), dim=0) > 0.97
