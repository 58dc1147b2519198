"""FP8 (E4M3, per-row scale) paged KV cache: quantizer properties, model-level agreement with the bf16 cache on CPU,
and the CUDA kernels (cache write, decode with in-kernel expansion, gather for prompt passes) against the PyTorch
restatement.  Reference: tests/test_kv_cache_quantized.py, tests/test_paged_attention_fp8.py."""
import pytest
import torch

from metal_marlin_b200 import ops
from metal_marlin_b200.models.mmfp4_causal_lm import MMFP4ForCausalLM

DEV = "cuda"


def test_fp8_pool_roundtrip_and_copy():
    p = ops.FP8KV(64, (2, 64), "cpu")
    rows = torch.randn(6, 2, 64) * 3
    idx = torch.tensor([1, 5, 9, 10, 33, 63])
    p.store(idx, rows)
    back = p[idx].float()
    # E4M3 keeps 3 mantissa bits: relative error of a value <= 2^-4, measured against the row maximum here
    assert float((back - rows).abs().max()) <= float(rows.abs().max()) * 0.0625 + 1e-6
    assert torch.all(p.scale[idx] > 0) and p.data.dtype == torch.uint8
    ops.kv_copy_rows(p, slice(16, 32), slice(0, 16))
    assert torch.equal(p[torch.tensor([17, 21])], p[torch.tensor([1, 5])])
    z = ops.FP8KV(4, (96,), "cpu")
    z.store(torch.tensor([2]), torch.zeros(1, 96))
    assert torch.all(z[torch.tensor([2])] == 0)


@pytest.mark.parametrize("preset", ["tiny-llama", "tiny-mla-moe"])
def test_generation_with_fp8_cache_tracks_bf16_cache_cpu(preset):
    lm = MMFP4ForCausalLM.from_config(preset, device="cpu", seed=3)
    prompts = [[5, 9, 200, 17, 3, 44, 8], [7, 7, 7, 12]]
    out_bf16 = lm.generate(prompts, max_new_tokens=6)
    out_fp8 = lm.generate(prompts, max_new_tokens=6, kv=lm.new_cache(16, 16, kv_dtype="fp8"))
    # greedy tokens of a random-init model are sensitive to tiny logit changes; the first generated token comes from the
    # prompt pass over freshly quantized rows and must agree, the rest must be valid ids
    for x, y in zip(out_bf16, out_fp8):
        assert x[0] == y[0] and len(x) == len(y)


@pytest.mark.gpu
@pytest.mark.parametrize("Hq,Hk,D", [(8, 2, 128), (4, 4, 64), (16, 2, 256)])
def test_fp8_cache_write_and_decode_kernels_gqa(Hq, Hk, D):
    torch.manual_seed(D)
    bs, ctxs = 16, [1, 70, 200]
    B = len(ctxs)
    nb = max((c + bs - 1) // bs for c in ctxs)
    bt = torch.randperm(B * nb, device=DEV).to(torch.int32).view(B, nb)
    kp, vp = ops.FP8KV(B * nb * bs, (Hk, D), DEV), ops.FP8KV(B * nb * bs, (Hk, D), DEV)
    kr, vr = ops.FP8KV(B * nb * bs, (Hk, D), DEV), ops.FP8KV(B * nb * bs, (Hk, D), DEV)
    inv = 1.0 / (1e4 ** (torch.arange(0, D, 2, device=DEV).float() / D))
    qn = (1 + 0.1 * torch.randn(D, device=DEV)).to(torch.bfloat16)
    kn = (1 + 0.1 * torch.randn(D, device=DEV)).to(torch.bfloat16)
    # fill the caches token by token through the prologue kernel (all sequences' tokens of one step per call)
    for step in range(max(ctxs)):
        live = [b for b in range(B) if step < ctxs[b]]
        T = len(live)
        qkv = (torch.randn(T, (Hq + 2 * Hk) * D, device=DEV) * 0.7).to(torch.bfloat16)
        pos = torch.full((T,), step, dtype=torch.int32, device=DEV)
        slots = torch.stack([bt[b, step // bs].long() * bs + step % bs for b in live])
        for pools, native in (((kp, vp), True), ((kr, vr), False)):
            x = qkv.clone()
            q, k, v = x[:, : Hq * D], x[:, Hq * D: (Hq + Hk) * D], x[:, (Hq + Hk) * D:]
            if native:
                ops.qk_norm_rope_cache(q, k, v, qn, kn, pos, inv, slots, pools[0], pools[1], Hq, Hk, D, 1e-6)
            else:
                with ops.force_reference():
                    ops.qk_norm_rope_cache(q, k, v, qn, kn, pos, inv, slots, pools[0], pools[1], Hq, Hk, D, 1e-6)
    used = torch.cat([bt[b, t // bs].long() * bs + t % bs for b in range(B) for t in [torch.arange(ctxs[b], device=DEV)]])
    # one E4M3 step of the row scale is the most the two quantizers may differ by
    dk = (kp[used].float() - kr[used].float()).abs().amax(-1)
    assert float((dk / (kr.scale[used] * 32 + 1e-6)).max()) <= 1.0
    cl = torch.tensor(ctxs, dtype=torch.int32, device=DEV)
    q = (torch.randn(B, Hq, D, device=DEV) * 0.5).to(torch.bfloat16)
    got = ops.paged_attention(q, kp, vp, bt, cl, Hq=Hq, Hkv=Hk, dqk=D, dv=D, block_size=bs, scale=D ** -0.5)
    with ops.force_reference():
        want = ops.paged_attention(q, kp, vp, bt, cl, Hq=Hq, Hkv=Hk, dqk=D, dv=D, block_size=bs, scale=D ** -0.5)
    torch.testing.assert_close(got.float(), want.float(), rtol=2e-2, atol=2e-2)
    # prompt pass over the quantized cache (gather kernel + contiguous attention)
    qn_tok = [1, 30, 64]
    qp = (torch.randn(sum(qn_tok), Hq, D, device=DEV) * 0.5).to(torch.bfloat16)
    cu_q = torch.tensor([0, 1, 31, 95], dtype=torch.int32, device=DEV)
    got = ops.prefill_attention(qp, kp, vp, cu_q, block_tables=bt, ctx_lens=cl, block_size=bs)
    with ops.force_reference():
        want = ops.prefill_attention(qp, kp, vp, cu_q, block_tables=bt, ctx_lens=cl, block_size=bs)
    torch.testing.assert_close(got.float(), want.float(), rtol=2e-2, atol=2e-2)


@pytest.mark.gpu
def test_fp8_latent_cache_mla_model_matches_reference_path():
    lm = MMFP4ForCausalLM.from_config("tiny-mla-moe", device="cuda", seed=5)
    prompts = [torch.randint(0, 512, (40,)).tolist(), torch.randint(0, 512, (9,)).tolist()]
    out = lm.generate(prompts, max_new_tokens=8, kv=lm.new_cache(16, 16, kv_dtype="fp8"))
    with ops.force_reference():
        ref = lm.generate(prompts, max_new_tokens=8, kv=lm.new_cache(16, 16, kv_dtype="fp8"), use_graph=False)
    assert [o[0] for o in out] == [r[0] for r in ref]
    agree = sum(a == b for o, r in zip(out, ref) for a, b in zip(o, r)) / sum(len(o) for o in out)
    assert agree >= 0.6, (out, ref)
