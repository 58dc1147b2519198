"""Hybrid stacks (Gated DeltaNet linear-attention layers or Mamba layers with periodic full-attention layers) on the shared decoder: state
handling across prefill, chunked prefill and decode, checkpoint round trip, the serving engine, and the CUDA kernels."""
import os

import pytest
import torch

from metal_marlin_b200 import ops
from metal_marlin_b200.engine.engine import EngineConfig, LLMEngine
from metal_marlin_b200.models.config import ModelConfig, get_preset
from metal_marlin_b200.models.mmfp4_causal_lm import MMFP4ForCausalLM, prefill


def test_layer_types_and_storage():
    cfg = get_preset("tiny-hybrid-deltanet")
    assert [cfg.layer_is_linear(i) for i in range(4)] == [True, True, True, False] and cfg.has_linear_layers
    d = cfg.to_dict()
    d.pop("layer_types")
    d["full_attention_interval"] = 4
    assert ModelConfig.from_dict(d).layer_types == cfg.layer_types                     # the interval form of HF configs
    lm = MMFP4ForCausalLM.from_config(cfg, device="cpu", seed=0)
    kv = lm.new_cache(8, 16)
    assert kv.k[0] is None and kv.k[3] is not None and kv.rec[3] is None
    conv, state = kv.rec[0]
    assert conv.shape == (8 + 1, 2 * 128 + 256, 3) and state.shape == (8 + 1, 8, 32, 32)        # + the parking entry of padded rows
    big = get_preset("qwen3.6-27b-hybrid")
    assert sum(big.layer_is_linear(i) for i in range(big.num_hidden_layers)) == 48


@pytest.mark.parametrize("preset", ["tiny-hybrid-deltanet", "tiny-jamba"])
def test_prefill_decode_and_chunking_agree_with_recomputation(preset):
    lm = MMFP4ForCausalLM.from_config(preset, device="cpu", seed=0)
    prompts = [list(range(3, 40)), [5, 6, 7, 8]]
    out = lm.generate(prompts, max_new_tokens=5)
    for pr, o in zip(prompts, out):            # every greedy token equals the arg-max of a from-scratch pass over the sequence
        seq = list(pr)
        for t in o:
            assert int(lm.forward_logits(seq)[-1].argmax()) == t
            seq.append(t)
    # chunked prefill carries the convolution window and the state matrix across chunks
    bt = torch.arange(8, dtype=torch.int32).view(2, 4)
    a = prefill(lm.model, lm.new_cache(8, 16), prompts, bt, chunk_tokens=4096)
    b = prefill(lm.model, lm.new_cache(8, 16), prompts, bt, chunk_tokens=7)
    assert float((a - b).abs().max() / a.abs().max()) < 2e-2
    # a cache slot that is reused by a new sequence starts from a clean state
    kv = lm.new_cache(8, 16)
    prefill(lm.model, kv, [prompts[0]], bt[:1])
    c = prefill(lm.model, kv, [prompts[1]], bt[:1])
    assert float((c[0] - a[1]).abs().max() / a[1].abs().max()) < 1e-2        # (a MoE layer may take another kernel path at another batch size)


@pytest.mark.parametrize("preset", ["tiny-hybrid-deltanet", "tiny-jamba"])
def test_checkpoint_roundtrip_and_engine(tmp_path, preset):
    from metal_marlin_b200.quant.convert import save_random_checkpoint
    cfg = get_preset(preset)
    out = str(tmp_path / "ck")
    info = save_random_checkpoint(cfg, out, fmt="mmfp4", seed=3)
    assert info["quantized"] > 0
    lm = MMFP4ForCausalLM.from_pretrained(out, device="cpu")
    assert lm.config.layer_types == cfg.layer_types
    if preset == "tiny-jamba":      # Mamba layers, one attention layer, MoE on every other layer
        assert lm.model.layers[0].mamba_in is not None and lm.model.layers[2].qkv is not None and lm.model.layers[2].router_w is not None
    else:
        assert lm.model.layers[0].lin_in is not None and lm.model.layers[3].qkv is not None
    prompts = [list(range(1, 30)), [9, 8, 7], list(range(40, 60))]
    want = [lm.generate([p], max_new_tokens=5)[0] for p in prompts]
    eng = LLMEngine(lm.model, EngineConfig(num_kv_blocks=32, block_size=16, max_model_len=64, max_chunk=16, max_prefill_tokens=32,
                                           use_cuda_graphs=False))
    assert eng.recurrent and not eng.cfg.enable_prefix_cache                     # state cannot be shared between sequences
    assert eng.generate(prompts, max_new_tokens=5) == want
    with pytest.raises(ValueError):
        eng.enable_speculative("ngram")
    from metal_marlin_b200.parallel.tp import shard_transformer
    with pytest.raises(NotImplementedError):
        shard_transformer(lm.model, 0, 2)


@pytest.mark.gpu
@pytest.mark.parametrize("preset", ["tiny-hybrid-deltanet", "tiny-jamba"])
def test_hybrid_model_on_the_gpu_matches_the_reference_path(preset):
    """Scan kernel (prompt), step kernel (decode, CUDA graph) and the FP4 kernels against the PyTorch restatement."""
    lm = MMFP4ForCausalLM.from_config(preset, device="cuda", seed=0)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 1024, (70,), generator=g).tolist(), torch.randint(0, 1024, (9,), generator=g).tolist()]
    bt = torch.arange(16, dtype=torch.int32).view(2, 8)
    a = prefill(lm.model, lm.new_cache(16, 16), prompts, bt)
    with ops.force_reference():
        b = prefill(lm.model, lm.new_cache(16, 16), prompts, bt)
    assert float((a - b).abs().max() / b.abs().max()) < 6e-2
    out_g = lm.generate(prompts, max_new_tokens=8, use_graph=True)
    out_e = lm.generate(prompts, max_new_tokens=8, use_graph=False)
    assert out_g == out_e and all(len(o) == 8 for o in out_g)
    with ops.force_reference():
        ref = lm.generate(prompts, max_new_tokens=8, use_graph=False)
    assert [o[0] for o in out_g] == [r[0] for r in ref]
    assert ops.check_status(torch.device("cuda")) == 0
