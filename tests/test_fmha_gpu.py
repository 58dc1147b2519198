"""Causal prefill attention on the tcgen05 kernel (``csrc/attention_fmha_sm100.cu``) against an fp32 PyTorch reference:
full prompts, ragged lengths, chunked prompts (queries are the last positions of the keys), grouped heads, strided
values, both head sizes, and score ranges that force the lazily deferred rescaling of the accumulator in tensor memory."""
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _ref(q, k, v, scale, window=0):
    t, Hq, D = q.shape
    n, Hk, _ = k.shape
    g = Hq // Hk
    qf, kf, vf = q.float(), k.float().repeat_interleave(g, 1), v.float().repeat_interleave(g, 1)
    s = torch.einsum("thd,nhd->htn", qf, kf) * scale
    pos = torch.arange(n - t, n, device=q.device).view(1, t, 1)
    keys = torch.arange(n, device=q.device).view(1, 1, n)
    s = s.masked_fill(keys > pos, float("-inf"))
    if window:
        s = s.masked_fill(keys <= pos - window, float("-inf"))
    return torch.einsum("htn,nhd->thd", torch.softmax(s, -1), vf)


@pytest.mark.parametrize("t,n,Hq,Hk,D,boost", [(512, 512, 4, 4, 256, 1.0), (300, 300, 8, 2, 256, 1.0), (256, 1000, 4, 1, 128, 1.0),
                                               (640, 640, 2, 2, 256, 8.0), (384, 900, 4, 2, 128, 8.0), (129, 129, 2, 2, 256, 1.0)])
def test_fmha_prefill_matches_reference(t, n, Hq, Hk, D, boost):
    from metal_marlin_b200 import ops
    torch.manual_seed(t + n)
    q = torch.randn(t, Hq, D, device=DEV).to(torch.bfloat16)
    k = torch.randn(n, Hk, D, device=DEV).to(torch.bfloat16)
    if boost != 1.0:          # later keys score far higher: the running maximum jumps by more than the lazy threshold
        k[n // 2:] *= boost
    kv = torch.randn(n, Hk, 2 * D, device=DEV).to(torch.bfloat16)
    v = kv[..., D:]           # strided rows, as the per-head values of the MLA prompt path are
    out = torch.empty(t, Hq, D, dtype=torch.bfloat16, device=DEV)
    scale = D ** -0.5
    ops.fmha_prefill(q, k, v, out, scale)
    torch.cuda.synchronize()
    assert ops.check_status(torch.device(DEV)) == 0
    ref = _ref(q, k, v, scale)
    err = float((out.float() - ref).abs().max() / ref.abs().max())
    assert err < 2e-2, err


@pytest.mark.parametrize("t,n,Hq,Hk,D,window", [(1024, 1024, 4, 2, 128, 64), (1024, 1536, 4, 2, 128, 300), (700, 900, 2, 2, 256, 100),
                                                (512, 2048, 2, 1, 256, 1000), (640, 640, 2, 2, 128, 4096), (384, 1200, 4, 4, 128, 1)])
def test_fmha_prefill_sliding_window(t, n, Hq, Hk, D, window):
    """Windows shorter than a key tile (a row's first visited tile can be wholly outside its window), longer than the
    context (no effect), and in between (leading key tiles are skipped)."""
    from metal_marlin_b200 import ops
    torch.manual_seed(t + n + window)
    q = torch.randn(t, Hq, D, device=DEV).to(torch.bfloat16)
    k = torch.randn(n, Hk, D, device=DEV).to(torch.bfloat16)
    v = torch.randn(n, Hk, D, device=DEV).to(torch.bfloat16)
    out = torch.empty(t, Hq, D, dtype=torch.bfloat16, device=DEV)
    scale = D ** -0.5
    ops.fmha_prefill(q, k, v, out, scale, window=window)
    torch.cuda.synchronize()
    assert ops.check_status(torch.device(DEV)) == 0
    ref = _ref(q, k, v, scale, window)
    err = float((out.float() - ref).abs().max() / ref.abs().max())
    assert err < 2e-2, err
    # the general entry point routes a windowed single sequence to the same kernel
    cu_q = torch.tensor([0, t], dtype=torch.int32, device=DEV)
    cu_k = torch.tensor([0, n], dtype=torch.int32, device=DEV)
    o2 = ops.prefill_attention(q, k, v, cu_q, cu_k=cu_k, max_q=t, window=window)
    assert float((o2.float() - ref).abs().max() / ref.abs().max()) < 2e-2


def test_prefill_attention_routes_single_sequences_to_the_tensor_core_kernel():
    from metal_marlin_b200 import ops
    torch.manual_seed(0)
    t, H, D = 512, 4, 256
    q, k, v = (torch.randn(t, H, D, device=DEV).to(torch.bfloat16) for _ in range(3))
    cu = torch.tensor([0, t], dtype=torch.int32, device=DEV)
    before = ops.launch_count()
    a = ops.prefill_attention(q, k, v, cu, cu_k=cu, max_q=t)
    with ops.force_reference():
        b = ops.prefill_attention(q, k, v, cu, cu_k=cu, max_q=t)
    assert float((a.float() - b.float()).abs().max() / b.float().abs().max()) < 2e-2
    assert ops.launch_count() > before


def test_mla_prompt_pass_with_tensor_core_attention_matches_reference():
    """A small MLA + MoE model with the head sizes of GLM-4.7-Flash (192 + 64 query / key, 256 value, latent 512): prompts
    of 256 and more tokens run keys-from-GEMM, V^T-from-GEMM and the tcgen05 attention kernel; a second, chunked pass
    attends over the cached first chunk."""
    import dataclasses
    from metal_marlin_b200 import ops
    from metal_marlin_b200.models.config import get_preset
    from metal_marlin_b200.models.mmfp4_causal_lm import MMFP4ForCausalLM, prefill
    cfg = dataclasses.replace(get_preset("tiny-mla-moe"), hidden_size=512, num_hidden_layers=2, kv_lora_rank=512, q_lora_rank=256,
                              qk_nope_head_dim=192, qk_rope_head_dim=64, v_head_dim=256)
    lm = MMFP4ForCausalLM.from_config(cfg, device="cuda", seed=3)
    prompts = [torch.randint(0, 512, (700,)).tolist(), torch.randint(0, 512, (301,)).tolist()]
    bt = torch.arange(2 * 48, dtype=torch.int32).view(2, 48)
    calls = {"n": 0}
    real = ops.fmha_prefill

    def counting(*a, **k):
        calls["n"] += 1
        return real(*a, **k)
    ops.fmha_prefill = counting
    try:
        a = prefill(lm.model, lm.new_cache(96, 16), prompts, bt)
    finally:
        ops.fmha_prefill = real
    assert calls["n"] == 2 * cfg.num_hidden_layers
    with ops.force_reference():
        b = prefill(lm.model, lm.new_cache(96, 16), prompts, bt)
    assert ops.check_status(torch.device(DEV)) == 0
    assert float((a - b).abs().max() / b.abs().max()) < 4e-2


def test_gqa_prompt_pass_with_tensor_core_attention_matches_reference():
    """Grouped-query model with 128-wide heads: one 600-token prompt, then a second chunk over the cached first one."""
    import dataclasses
    from metal_marlin_b200 import ops
    from metal_marlin_b200.models.config import get_preset
    from metal_marlin_b200.models.mmfp4_causal_lm import MMFP4ForCausalLM, prefill
    cfg = dataclasses.replace(get_preset("tiny-qwen3-moe"), head_dim=128, num_attention_heads=4, num_key_value_heads=2, hidden_size=512)
    lm = MMFP4ForCausalLM.from_config(cfg, device="cuda", seed=4)
    prompts = [torch.randint(0, 512, (600,)).tolist()]
    bt = torch.arange(48, dtype=torch.int32).view(1, 48)
    calls = {"n": 0}
    real = ops.fmha_prefill

    def counting(*a, **k):
        calls["n"] += 1
        return real(*a, **k)
    ops.fmha_prefill = counting
    try:
        a = prefill(lm.model, lm.new_cache(48, 16), prompts, bt)
    finally:
        ops.fmha_prefill = real
    assert calls["n"] == cfg.num_hidden_layers
    with ops.force_reference():
        b = prefill(lm.model, lm.new_cache(48, 16), prompts, bt)
    assert ops.check_status(torch.device(DEV)) == 0
    assert float((a - b).abs().max() / b.abs().max()) < 4e-2


def test_gqa_batch_of_long_prompts_runs_the_tensor_core_attention_per_sequence():
    """Several long prompts in one pass: the tcgen05 kernel is launched once per sequence and layer (not the mma.sync kernel for
    the whole batch); a short prompt in the batch sends the pass back to the batched kernel."""
    import dataclasses
    from metal_marlin_b200 import ops
    from metal_marlin_b200.models.config import get_preset
    from metal_marlin_b200.models.mmfp4_causal_lm import MMFP4ForCausalLM, prefill
    cfg = dataclasses.replace(get_preset("tiny-qwen3-moe"), head_dim=128, num_attention_heads=4, num_key_value_heads=2, hidden_size=512)
    lm = MMFP4ForCausalLM.from_config(cfg, device="cuda", seed=4)
    prompts = [torch.randint(0, 512, (n,)).tolist() for n in (600, 257, 431)]
    bt = torch.arange(3 * 48, dtype=torch.int32).view(3, 48)
    calls = {"n": 0}
    real = ops.fmha_prefill

    def counting(*a, **k):
        calls["n"] += 1
        return real(*a, **k)
    ops.fmha_prefill = counting
    try:
        a = prefill(lm.model, lm.new_cache(3 * 48, 16), prompts, bt)
        assert calls["n"] == 3 * cfg.num_hidden_layers
        calls["n"] = 0
        mixed = prefill(lm.model, lm.new_cache(3 * 48, 16), prompts[:2] + [[5, 6, 7]], bt)
        assert calls["n"] == 0 and torch.isfinite(mixed).all()
    finally:
        ops.fmha_prefill = real
    with ops.force_reference():
        b = prefill(lm.model, lm.new_cache(3 * 48, 16), prompts, bt)
    assert ops.check_status(torch.device(DEV)) == 0
    assert float((a - b).abs().max() / b.abs().max()) < 4e-2


def test_sliding_window_model_prompts_take_the_tensor_core_kernel():
    """A grouped-query model with a 200-token window: a 700-token prompt, then a 300-token continuation over the cached
    keys (only the keys inside the chunk's window are gathered), against the PyTorch restatement of every op."""
    import dataclasses
    from metal_marlin_b200 import ops
    from metal_marlin_b200.models.config import get_preset
    from metal_marlin_b200.models.mmfp4_causal_lm import MMFP4ForCausalLM, prefill
    cfg = dataclasses.replace(get_preset("tiny-llama"), hidden_size=512, num_attention_heads=4, num_key_value_heads=2, head_dim=128,
                              sliding_window=200)
    lm = MMFP4ForCausalLM.from_config(cfg, device="cuda", seed=5)
    g = torch.Generator().manual_seed(9)
    seq = torch.randint(0, cfg.vocab_size, (1000,), generator=g).tolist()
    bt = torch.arange(64, dtype=torch.int32).view(1, 64)
    calls = {"n": 0}
    real = ops.fmha_prefill

    def counting(*a, **k):
        calls["n"] += 1
        assert k.get("window") == 200
        return real(*a, **k)
    ops.fmha_prefill = counting
    try:
        kv = lm.new_cache(64, 16)
        prefill(lm.model, kv, [seq[:700]], bt)
        a = prefill(lm.model, kv, [seq], bt, start=[700])
    finally:
        ops.fmha_prefill = real
    assert calls["n"] == 2 * cfg.num_hidden_layers
    assert ops.check_status(torch.device(DEV)) == 0
    with ops.force_reference():
        kv = lm.new_cache(64, 16)
        prefill(lm.model, kv, [seq[:700]], bt)
        b = prefill(lm.model, kv, [seq], bt, start=[700])
    err = float((a - b).abs().max() / b.abs().max())
    assert err < 5e-2, err


@pytest.mark.parametrize("kv_dtype,window", [("fp8", 0), ("int8", 200), ("fp4", 0)])
def test_quantized_cache_prompts_take_the_tensor_core_kernel(kv_dtype, window):
    """Grouped-query model over a quantized paged cache: the rows of a sequence are expanded by the cache's gather kernel
    and the prompt attention runs on the tcgen05 kernel (first pass and a chunk over cached keys, optionally windowed)."""
    import dataclasses
    from metal_marlin_b200 import ops
    from metal_marlin_b200.models.config import get_preset
    from metal_marlin_b200.models.mmfp4_causal_lm import MMFP4ForCausalLM, prefill
    cfg = dataclasses.replace(get_preset("tiny-llama"), hidden_size=512, num_attention_heads=4, num_key_value_heads=2, head_dim=128,
                              sliding_window=window)
    lm = MMFP4ForCausalLM.from_config(cfg, device="cuda", seed=6)
    g = torch.Generator().manual_seed(10)
    seqs = [torch.randint(0, cfg.vocab_size, (900,), generator=g).tolist(), torch.randint(0, cfg.vocab_size, (860,), generator=g).tolist()]
    bt = torch.arange(2 * 64, dtype=torch.int32).view(2, 64)
    calls = {"n": 0}
    real = ops.fmha_prefill

    def counting(*a, **k):
        calls["n"] += 1
        return real(*a, **k)
    ops.fmha_prefill = counting
    try:
        kv = lm.new_cache(128, 16, kv_dtype=kv_dtype)
        prefill(lm.model, kv, [s[:600] for s in seqs], bt)
        a = prefill(lm.model, kv, seqs, bt, start=[600, 600])
    finally:
        ops.fmha_prefill = real
    assert calls["n"] == 2 * 2 * cfg.num_hidden_layers          # two passes x two sequences x layers
    assert ops.check_status(torch.device(DEV)) == 0
    with ops.force_reference():
        kv = lm.new_cache(128, 16, kv_dtype=kv_dtype)
        prefill(lm.model, kv, [s[:600] for s in seqs], bt)
        b = prefill(lm.model, kv, seqs, bt, start=[600, 600])
    err = float((a - b).abs().max() / b.abs().max())
    assert err < (0.25 if kv_dtype == "fp4" else 8e-2), err
