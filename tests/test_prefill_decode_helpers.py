"""Prompt-pass and decode helpers (``inference/prefill.py``, ``inference/decode.py``) on the CPU restatement: chunking and
its statistics, chunk sizing from a memory budget, bulk KV writes, the layout wrapper of the prompt attention, speculative
prefill, the persistent decode state against step-by-step generation, kernel selection and quantized-cache attention.
Parity: reference ``tests/test_prefill.py`` / ``tests/test_decode.py`` (same surfaces on its caches)."""
import dataclasses

import pytest
import torch

from metal_marlin_b200 import ops
from metal_marlin_b200.inference import decode as dec
from metal_marlin_b200.inference import prefill as pre
from metal_marlin_b200.models.config import get_preset
from metal_marlin_b200.models.mmfp4_causal_lm import MMFP4ForCausalLM, prefill


@pytest.fixture(scope="module")
def lm():
    return MMFP4ForCausalLM.from_config(get_preset("tiny-llama"), device="cpu", seed=1)


def test_chunked_prefill_matches_single_pass_and_reports(lm):
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, 1024, (150,), generator=g).tolist()
    seen = []
    logits, stats, kv, bt = pre.chunked_prefill(lm, ids, config=pre.PrefillConfig(chunk_size=64),
                                                progress_callback=lambda a, b: seen.append((a, b)))
    assert stats.num_chunks == 3 and stats.total_tokens == 150 and len(stats.chunk_times_ms) == 3
    assert seen == [(64, 150), (128, 150), (150, 150)] and stats.tokens_per_second > 0
    kv2 = lm.new_cache(bt.shape[1], 16)
    ref = prefill(lm.model, kv2, [ids], bt)[0]
    assert float((logits - ref).abs().max()) < 2e-2 * float(ref.abs().max())
    with pytest.raises(ValueError):
        pre.chunked_prefill(lm, ids, kv=kv, block_table=bt[:, :4])


def test_pick_chunk_size_follows_the_memory_budget():
    cfg = get_preset("glm-4.7-flash")
    auto = pre.PrefillConfig(chunk_size=0)
    big = pre.pick_chunk_size(cfg, 32768, auto, free_bytes=100 << 30)
    small = pre.pick_chunk_size(cfg, 32768, auto, free_bytes=3 << 30)
    assert big == 32768 and auto.min_chunk <= small < big
    assert pre.estimate_chunk_bytes(cfg, small, 32768) <= 0.8 * (3 << 30) or small == auto.min_chunk
    assert pre.pick_chunk_size(cfg, 100, pre.PrefillConfig(chunk_size=512)) == 512


def test_parallel_kv_write_bf16_and_quantized(lm):
    cfg = lm.model.cfg
    slots = torch.tensor([3, 17, 40])
    rows = [(li, torch.randn(3, cfg.num_key_value_heads, cfg.dh), torch.randn(3, cfg.num_key_value_heads, cfg.dh)) for li in range(2)]
    kv = lm.new_cache(4, 16)
    pre.parallel_kv_write(kv, rows, slots)
    assert torch.equal(kv.k[1][slots].float(), rows[1][1].to(torch.bfloat16).float())
    assert float(kv.v[0][5].abs().max()) == 0.0
    kq = lm.new_cache(4, 16, kv_dtype="fp8")
    pre.parallel_kv_write(kq, rows, slots)
    got = kq.k[0][slots].float()
    assert float((got - rows[0][1]).abs().max()) < 0.08 * float(rows[0][1].abs().max())


def test_flash_prefill_attention_layout():
    torch.manual_seed(0)
    B, Hq, Hk, T, N, D = 2, 4, 2, 5, 9, 64
    q, k, v = torch.randn(B, Hq, T, D), torch.randn(B, Hk, N, D), torch.randn(B, Hk, N, D)
    out = pre.flash_prefill_attention(q.bfloat16(), k.bfloat16(), v.bfloat16()).float()
    kk, vv = k.repeat_interleave(2, 1), v.repeat_interleave(2, 1)
    s = torch.einsum("bhtd,bhnd->bhtn", q, kk) * D ** -0.5
    mask = torch.arange(N).view(1, N) > (torch.arange(T).view(T, 1) + N - T)
    ref = torch.softmax(s.masked_fill(mask, float("-inf")), -1) @ vv
    assert out.shape == (B, Hq, T, D) and float((out - ref).abs().max()) < 3e-2
    one = pre.flash_prefill_attention(q[:1].bfloat16(), k[:1].bfloat16(), v[:1].bfloat16(), window=3).float()
    mask3 = mask | (torch.arange(N).view(1, N) <= (torch.arange(T).view(T, 1) + N - T - 3))
    ref3 = torch.softmax(s[:1].masked_fill(mask3, float("-inf")), -1) @ vv[:1]
    assert float((one - ref3).abs().max()) < 3e-2


def test_speculative_prefill_extends_the_cache_only_when_confident(lm):
    ids = list(range(5, 45))
    bt = torch.arange(4, dtype=torch.int32).view(1, 4)
    base, none = pre.speculative_prefill(lm, ids, lm.new_cache(4, 16), bt)
    assert none == []
    lg, spec = pre.speculative_prefill(lm, ids, lm.new_cache(4, 16), bt,
                                       pre.SpeculativePrefillConfig(enabled=True, num_speculative_tokens=3, confidence_threshold=0.0))
    assert len(spec) == 3 and spec[0] == int(base.argmax())
    full = prefill(lm.model, lm.new_cache(4, 16), [ids + spec], bt)[0]
    assert float((lg - full).abs().max()) < 2e-2 * float(full.abs().max())
    _, shy = pre.speculative_prefill(lm, ids, lm.new_cache(4, 16), bt,
                                     pre.SpeculativePrefillConfig(enabled=True, confidence_threshold=0.999))
    assert shy == []


def test_decode_state_reproduces_greedy_generation(lm):
    prompts = [list(range(3, 20)), list(range(100, 110))]
    st = dec.DecodeState(lm, dec.DecodeConfig(batch_size=2, max_context=64, max_new_tokens=6))
    first = st.prefill(prompts)
    toks = [first.clone()]
    for _ in range(5):
        toks.append(dec.persistent_decode_step(st, timed=True).clone())
    got = torch.stack(toks, 1)
    ref = lm.generate(prompts, max_new_tokens=6)
    assert got.tolist() == [list(r) for r in ref]          # generate returns the new tokens only
    assert len(st.stats.step_times_ms) == 5 and st.stats.tokens_per_second > 0 and st.stats.weight_read_mb > 0
    assert st.lengths == [22, 15]


def test_select_decode_kernel_follows_thresholds():
    assert dec.select_decode_kernel(1, 4096, 4096) == "fp4_gemv_fused_prologue"
    assert dec.select_decode_kernel(16, 4096, 4096).startswith("fp4_gemv")
    assert dec.select_decode_kernel(64, 4096, 4096) == "fp4_gemm_tcgen05"
    old = dict(ops.GEMV_LIMITS)
    try:
        ops.GEMV_LIMITS = {(4096, 4096): 128}
        assert dec.select_decode_kernel(64, 4096, 4096).startswith("fp4_gemv")
    finally:
        ops.GEMV_LIMITS = old


@pytest.mark.parametrize("fmt,tol", [("fp8", 0.06), ("int8", 0.02), ("fp4", 0.35), ("int4", 0.3)])
def test_quantized_kv_attention_contiguous_layout(fmt, tol):
    torch.manual_seed(1)
    B, Hq, Hk, S, D = 2, 4, 2, 37, 64
    q = torch.randn(B, Hq, 1, D).bfloat16()
    k, v = torch.randn(B, Hk, S, D), torch.randn(B, Hk, S, D)
    kc, ks = dec.quantize_kv_cache(k, fmt)
    vc, vs = dec.quantize_kv_cache(v, fmt)
    assert kc.shape == (B, Hk, S, D // 2 if fmt in ("fp4", "int4") else D) and ks.shape == (B, Hk, S)
    lens = torch.tensor([S, 20], dtype=torch.int32)
    out = dec.quantized_kv_attention(q, kc, vc, ks, vs, Hq, Hk, seq_lens=lens, quant_dtype=fmt).float()
    ref = torch.zeros(B, Hq, 1, D)
    for b in range(B):
        n = int(lens[b])
        kk, vv = k[b, :, :n].repeat_interleave(2, 0), v[b, :, :n].repeat_interleave(2, 0)
        p = torch.softmax(torch.einsum("hqd,hnd->hqn", q[b].float(), kk) * D ** -0.5, -1)
        ref[b] = p @ vv
    assert float((out - ref).abs().max()) < tol * float(ref.abs().max()) + 0.02


def test_fused_sampling_and_allocation_free_generate_loop():
    """Reference ``tests/test_fused_sampling_optimized.py`` / ``test_optimized_generate.py``."""
    import types
    import torch
    from metal_marlin_b200.inference import _fused_sampling, _optimized_generate
    p = torch.tensor([[0.1, 0.6, 0.3], [0.7, 0.2, 0.1]])
    assert _fused_sampling(p, temperature=0.0).tolist() == [[1], [0]]
    out = torch.zeros(2, 1, dtype=torch.int64)
    assert _fused_sampling(p, temperature=1.0, top_k=1, out=out) is out and out.tolist() == [[1], [0]]
    draws = torch.cat([_fused_sampling(p[:1], temperature=1.0, top_p=0.5, seed=3) for _ in range(60)])
    assert set(draws.reshape(-1).tolist()) == {1}                                       # the nucleus of 0.5 holds one token
    two = torch.cat([_fused_sampling(p[:1], temperature=1.0, top_p=0.65, seed=4) for _ in range(200)])
    assert set(two.reshape(-1).tolist()) == {1, 2}                                      # 0.6 < 0.65: the next token joins the nucleus
    wide = torch.cat([_fused_sampling(p[:1], temperature=1.0, top_p=1.0, seed=5) for _ in range(200)]).reshape(-1)
    assert set(wide.tolist()) == {0, 1, 2} and (wide == 1).sum() > (wide == 0).sum()

    V = 11

    class Toy:
        """Next token = (last token + 1) mod V; with a cache it must be fed one token at a time."""
        def __init__(self, cache=True):
            self.cache, self.calls = cache, []

        def __call__(self, input_ids=None, past_key_values=None, use_cache=True, attention_mask=None):
            self.calls.append((tuple(input_ids.shape), None if attention_mask is None else attention_mask.shape[1]))
            logits = torch.full((*input_ids.shape, V), -10.0)
            logits.scatter_(2, ((input_ids + 1) % V).unsqueeze(-1), 10.0)
            past = (0 if past_key_values is None else past_key_values) + input_ids.shape[1] if self.cache else None
            return types.SimpleNamespace(logits=logits, past_key_values=past)
    ids = torch.tensor([[3, 4], [8, 9]])
    m = Toy()
    seq, past = _optimized_generate(m, ids, 4, temperature=0.0, return_past_key_values=True, attention_mask=torch.ones_like(ids))
    assert seq.tolist() == [[3, 4, 5, 6, 7, 8], [8, 9, 10, 0, 1, 2]] and past == 5
    assert [c[0] for c in m.calls] == [(2, 2), (2, 1), (2, 1), (2, 1)] and [c[1] for c in m.calls] == [2, 3, 4, 5]
    nocache = Toy(cache=False)
    assert _optimized_generate(nocache, ids, 2, temperature=0.0).tolist() == [[3, 4, 5, 6], [8, 9, 10, 0]] and nocache.calls[1][0] == (2, 3)
    stop = _optimized_generate(Toy(), ids, 6, temperature=0.0, eos_token_id=6, pad_token_id=99)
    assert stop[0].tolist()[:4] == [3, 4, 5, 6] and (stop[0, 4:] == 99).all() and stop.shape[1] == 8      # row 1 never stops: the loop runs on
    both = _optimized_generate(Toy(), torch.tensor([[4], [4]]), 6, temperature=0.0, eos_token_id=6)
    assert both.tolist() == [[4, 5, 6], [4, 5, 6]]                                     # every row done: early exit
    sampled = _optimized_generate(Toy(), ids, 3, temperature=0.7, top_p=0.9, top_k=3, seed=1)
    assert sampled.tolist() == [[3, 4, 5, 6, 7], [8, 9, 10, 0, 1]]                      # the peaked toy distribution leaves one choice
