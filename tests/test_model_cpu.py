"""CPU reference path: decode equals prefill, generation is deterministic, configs parse."""
import json

import pytest
import torch

from metal_marlin_b200.models.config import ModelConfig, get_preset, glm47_flash
from metal_marlin_b200.models.mmfp4_causal_lm import MMFP4ForCausalLM


@pytest.mark.parametrize("preset", ["tiny-llama", "tiny-mla-moe", "tiny-qwen3-moe"])
def test_incremental_decode_equals_full_prefill(preset):
    lm = MMFP4ForCausalLM.from_config(preset, device="cpu", seed=0)
    prompt = torch.randint(0, lm.config.vocab_size, (21,)).tolist()
    out = lm.generate([prompt], max_new_tokens=6)[0]
    # teacher-forced logits over prompt + generated must pick the same tokens greedily
    full = lm.forward_logits(prompt + out[:-1])
    greedy = full[len(prompt) - 1:].argmax(-1).tolist()
    assert greedy == out


def test_tiny_llama_workload_shape():
    """Config 1: 2 layers, hidden 256, 4 heads x 64, SwiGLU 688, vocab 1024; 16 prompt ids -> 32 tokens."""
    lm = MMFP4ForCausalLM.from_config("tiny-llama", device="cpu", seed=0)
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, 1024, (16,), generator=g).tolist()
    a = lm.generate([prompt], max_new_tokens=32)[0]
    b = lm.generate([prompt], max_new_tokens=32)[0]
    assert a == b and len(a) == 32


def test_batch_generation_independent_of_batch_mates():
    lm = MMFP4ForCausalLM.from_config("tiny-mla-moe", device="cpu", seed=1)
    p1, p2 = list(range(3, 30)), list(range(100, 108))
    solo = lm.generate([p1], max_new_tokens=5)[0]
    both = lm.generate([p1, p2], max_new_tokens=5)
    assert both[0] == solo


def test_glm47_flash_dimensions():
    cfg = glm47_flash()
    pc = cfg.param_count()
    assert cfg.latent_dim == 576 and cfg.qk_head_dim == 256
    assert 29e9 < pc["total"] < 31e9          # ~30 B total
    assert 2.5e9 < pc["active"] < 3.6e9       # ~3 B active per token


def test_config_from_hf_dict_aliases(tmp_path):
    d = {"model_type": "glm4_moe_lite", "text_config": {"hidden_size": 64, "n_routed_experts": 8, "num_experts_per_tok": 2,
         "kv_lora_rank": 16, "qk_rope_head_dim": 8, "qk_nope_head_dim": 8, "v_head_dim": 8, "num_hidden_layers": 2,
         "num_attention_heads": 2, "vocab_size": 100, "moe_intermediate_size": 32, "intermediate_size": 64},
         "quantization_config": {"format": "mmfp4_e2m1_marlin", "group_size": 32}}
    (tmp_path / "config.json").write_text(json.dumps(d))
    cfg = ModelConfig.from_pretrained(str(tmp_path))
    assert cfg.num_experts == 8 and cfg.is_mla and cfg.group_size == 32 and cfg.quant_format == "mmfp4"
    assert cfg.scoring_func == "sigmoid" and cfg.rope_interleave


def test_eager_bf16_baseline_tracks_the_model():
    """The eager bf16 baseline wrapper runs prefill + decode and stays close to the fp32-restatement logits."""
    from metal_marlin_b200.baseline_eager import EagerBF16Model
    from metal_marlin_b200.engine.session import DecodeSession, SamplingParams
    from metal_marlin_b200.models.mmfp4_causal_lm import MMFP4ForCausalLM, prefill
    lm = MMFP4ForCausalLM.from_config("tiny-mla-moe", device="cpu", seed=2)
    em = EagerBF16Model(lm.model)
    prompts = [list(range(5, 30))]
    bt = torch.arange(4, dtype=torch.int32).view(1, 4)
    kv_a, kv_b = lm.new_cache(4, 16), lm.new_cache(4, 16)
    lg_ref = prefill(lm.model, kv_a, prompts, bt)
    lg_eager = em.prefill(kv_b, prompts, bt)
    assert (lg_ref - lg_eager).abs().max() / lg_ref.abs().max() < 0.1
    sess = DecodeSession(em, kv_b, 1, 4, max_new_tokens=4, use_graph=False)
    sess.set_sampling([SamplingParams()])
    sess.set_state(lg_eager.argmax(-1), [25], bt)
    toks = [int(sess.step()[0]) for _ in range(3)]
    assert all(0 <= t < lm.config.vocab_size for t in toks)


def test_kv_b_split_cache_follows_a_sharded_copy_of_the_layer():
    """The prompt path caches the key / value halves of ``kv_b`` on the layer object; a shallow copy of the layer whose
    matrix was sliced for tensor parallelism (rank 0's slice starts at the same address) must get its own split."""
    import copy
    from metal_marlin_b200.models.mmfp4_causal_lm import MMFP4ForCausalLM
    lm = MMFP4ForCausalLM.from_config("tiny-mla-moe", device="cpu", seed=1)
    m, cfg = lm.model, lm.config
    L = m.layers[0]
    H, dn, dv, R = m.n_heads_local, cfg.qk_nope_head_dim, cfg.v_head_dim, cfg.kv_lora_rank
    w_k, w_v = m._kv_b_split(L)
    assert w_k.shape == (H * dn, R) and w_v.shape == (H, dv, R)
    S = copy.copy(L)
    S.kv_b_dense = L.kv_b_dense[: (H // 2) * (dn + dv)].contiguous()
    assert S.kv_b_dense.data_ptr() == L.kv_b_dense.data_ptr()
    m2 = copy.copy(m)
    m2.n_heads_local = H // 2
    w_k2, w_v2 = m2._kv_b_split(S)
    assert w_k2.shape == ((H // 2) * dn, R) and w_v2.shape == (H // 2, dv, R)
    full = L.kv_b_dense.view(H, dn + dv, R)
    assert torch.equal(w_k2, full[: H // 2, :dn].reshape(-1, R)) and torch.equal(w_v2, full[: H // 2, dn:])
