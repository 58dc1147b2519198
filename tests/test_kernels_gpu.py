"""Numerics of every sm_100a kernel against the plain-PyTorch fp32 restatement of the same op.
Shapes follow the reference's tests/test_gemm.py (tile-boundary M/N/K, group sizes, zero input,
determinism) and tests/test_paged_attention*.py / test_mla_fused.py / test_sampling*.py."""
import math

import pytest
import torch

from metal_marlin_b200 import ops
from metal_marlin_b200.ops import FP4ExpertBank, FP4Weight
from metal_marlin_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _close(a, b, rtol=2e-2, atol=2e-2):
    a, b = a.float(), b.float()
    err = (a - b).abs()
    tol = atol * b.abs().max().clamp_min(1e-6) + rtol * b.abs()
    assert bool((err <= tol).all()), f"max err {err.max().item():.4g}, ref max {b.abs().max().item():.4g}"


def _bf(*shape, scale=1.0):
    return (torch.randn(*shape, device=DEV) * scale).to(torch.bfloat16)


def test_native_library_loaded():
    assert ops.native_available()
    assert hasattr(torch.ops.mmb200, "fp4_gemv")


@pytest.mark.parametrize("M", [1, 2, 7, 8, 11, 16, 17, 25, 32])        # above 8 tokens: 2 / 4 row blocks per CTA
@pytest.mark.parametrize("N,K,gs", [(768, 2048, 128), (2048, 5120, 128), (576, 768, 128), (48, 192, 64), (16, 64, 32),
                                    (1344, 2048, 128), (9472, 2048, 128)])
def test_fp4_gemv_matches_reference(M, N, K, gs):
    torch.manual_seed(M * 1000 + N)
    W = FP4Weight.from_float(torch.randn(N, K, device=DEV) * 0.02, gs)
    x = _bf(M, K)
    y = ops.linear(x, W)
    with ops.force_reference():
        y_ref = ops.linear(x, W)
    _close(y, y_ref, rtol=1e-2, atol=4e-3)


def test_fp4_gemv_exact_on_integer_problem():
    # integer activations x E2M1 codes x power-of-two scales: every product and sum is exact in fp32
    N, K = 64, 256
    codes = torch.randint(0, 16, (N, K), dtype=torch.uint8, device=DEV)
    scales = torch.full((N, K // 128), 0.5, dtype=torch.float16, device=DEV)
    W = FP4Weight.from_codes(codes, scales)
    x = torch.randint(-3, 4, (3, K), device=DEV).to(torch.bfloat16)
    y = ops.linear(x, W).float()
    y_ref = x.float() @ W.dequantize().t()
    assert torch.equal(y, y_ref.to(torch.bfloat16).float())


def test_fp4_gemv_zero_input_and_determinism():
    W = FP4Weight.from_float(torch.randn(256, 512, device=DEV), 128)
    assert torch.all(ops.linear(torch.zeros(2, 512, device=DEV, dtype=torch.bfloat16), W) == 0)
    x = _bf(4, 512)
    assert torch.equal(ops.linear(x, W), ops.linear(x, W))


@pytest.mark.parametrize("M", [1, 5, 16, 27, 32])
def test_fp4_gemv_fused_prologue_epilogue(M):
    K, N = 1024, 512
    W = FP4Weight.from_float(torch.randn(N, K, device=DEV) * 0.03, 128)
    x, d, nw = _bf(M, K), _bf(M, K, scale=0.3), (1 + 0.1 * torch.randn(K, device=DEV)).to(torch.bfloat16)
    bias, add = _bf(N, scale=0.1), _bf(M, N)
    r1, r2 = torch.empty_like(x), torch.empty_like(x)
    y = ops.linear(x, W, delta=d, norm_w=nw, eps=1e-5, resid_out=r1, bias=bias, out_add=add)
    with ops.force_reference():
        y_ref = ops.linear(x, W, delta=d, norm_w=nw, eps=1e-5, resid_out=r2, bias=bias, out_add=add)
    assert torch.equal(r1, r2)
    _close(y, y_ref, rtol=1e-2, atol=5e-3)
    # SwiGLU epilogue over the two row halves
    g = ops.linear(x, W, norm_w=nw, act=1)
    with ops.force_reference():
        g_ref = ops.linear(x, W, norm_w=nw, act=1)
    assert g.shape == (M, N // 2)
    _close(g, g_ref, rtol=2e-2, atol=5e-3)


def test_fp4_gemv_strided_input_slice():
    K, N = 768, 256
    W = FP4Weight.from_float(torch.randn(N, K, device=DEV) * 0.03, 128)
    buf = _bf(3, 1344)
    nw = torch.ones(K, device=DEV, dtype=torch.bfloat16)
    y = ops.linear(buf[:, :K], W, norm_w=nw)
    with ops.force_reference():
        y_ref = ops.linear(buf[:, :K], W, norm_w=nw)
    _close(y, y_ref, rtol=1e-2, atol=5e-3)


@pytest.mark.parametrize("T,E,topk,ns", [(1, 8, 2, 1), (4, 64, 4, 1), (3, 16, 8, 0), (9, 8, 2, 2)])
def test_moe_gemv_path(T, E, topk, ns):
    H, I = 256, 128
    gu = FP4ExpertBank.from_float(torch.randn(E + ns, 2 * I, H, device=DEV) * 0.05, 64)
    dn = FP4ExpertBank.from_float(torch.randn(E + ns, H, I, device=DEV) * 0.05, 64)
    x = _bf(T, H)
    nw = (1 + 0.1 * torch.randn(H, device=DEV)).to(torch.bfloat16)
    ids = torch.stack([torch.randperm(E, device=DEV)[:topk] for _ in range(T)]).to(torch.int32)
    wts = torch.rand(T, topk, device=DEV)
    add = _bf(T, H)
    h = ops.moe_gate_up(x, gu, ids, n_shared=ns, shared_base=E, norm_w=nw)
    y = ops.moe_down(h, dn, ids, wts, n_shared=ns, shared_base=E, out_add=add)
    with ops.force_reference():
        h_ref = ops.moe_gate_up(x, gu, ids, n_shared=ns, shared_base=E, norm_w=nw)
        y_ref = ops.moe_down(h_ref, dn, ids, wts, n_shared=ns, shared_base=E, out_add=add)
    _close(h, h_ref, rtol=2e-2, atol=5e-3)
    _close(y, y_ref, rtol=2e-2, atol=1e-2)


@pytest.mark.parametrize("M,N,K", [(1, 1000, 256), (4, 64, 2048), (8, 333, 512), (20, 128, 256)])
def test_bf16_gemv(M, N, K):
    w, x = _bf(N, K, scale=0.05), _bf(M, K)
    nw = (1 + 0.1 * torch.randn(K, device=DEV)).to(torch.bfloat16)
    d = _bf(M, K, scale=0.2)
    y = ops.bf16_linear(x, w, delta=d, norm_w=nw, out_dtype=torch.float32)
    with ops.force_reference():
        y_ref = ops.bf16_linear(x, w, delta=d, norm_w=nw, out_dtype=torch.float32)
    _close(y, y_ref, rtol=5e-3, atol=2e-3)


@pytest.mark.parametrize("rows,dim", [(1, 2048), (5, 768), (3, 64), (2, 10240)])
def test_rmsnorm(rows, dim):
    x, d = _bf(rows, dim), _bf(rows, dim)
    w = (1 + 0.1 * torch.randn(dim, device=DEV)).to(torch.bfloat16)
    r1, r2 = torch.empty_like(x), torch.empty_like(x)
    y = ops.rmsnorm(x, w, 1e-5, delta=d, resid_out=r1)
    with ops.force_reference():
        y_ref = ops.rmsnorm(x, w, 1e-5, delta=d, resid_out=r2)
    assert torch.equal(r1, r2)
    _close(y, y_ref, rtol=1e-2, atol=1e-3)


def test_rmsnorm_large_values_no_overflow():
    x = torch.full((1, 4096), 30000.0, device=DEV, dtype=torch.bfloat16)
    y = ops.rmsnorm(x, torch.ones(4096, device=DEV, dtype=torch.bfloat16), 1e-6)
    assert torch.isfinite(y.float()).all() and abs(float(y[0, 0]) - 1.0) < 1e-2


def test_silu_mul_and_embedding():
    gu = _bf(7, 512)
    with ops.force_reference():
        r = ops.silu_mul(gu)
    _close(ops.silu_mul(gu), r, rtol=1e-2, atol=1e-3)
    table = _bf(100, 64)
    ids = torch.randint(0, 100, (9,), device=DEV)
    assert torch.equal(ops.embedding(table, ids), table[ids])


@pytest.mark.parametrize("interleaved", [False, True])
def test_qk_norm_rope_cache(interleaved):
    T, Hq, Hk, D = 6, 8, 2, 128
    qkv = _bf(T, (Hq + 2 * Hk) * D)
    qkv2 = qkv.clone()
    qn, kn = (1 + 0.1 * torch.randn(D, device=DEV)).to(torch.bfloat16), (1 + 0.1 * torch.randn(D, device=DEV)).to(torch.bfloat16)
    pos = torch.tensor([0, 1, 2, 40, 41, 1000], dtype=torch.int32, device=DEV)
    inv = 1.0 / (10000 ** (torch.arange(0, D, 2, device=DEV).float() / D))
    slots = torch.tensor([3, 4, 5, 20, -1, 7], device=DEV)
    kp, vp = torch.zeros(32, Hk, D, device=DEV, dtype=torch.bfloat16), torch.zeros(32, Hk, D, device=DEV, dtype=torch.bfloat16)
    kp2, vp2 = kp.clone(), vp.clone()

    def run(buf, k_pool, v_pool):
        q, k, v = buf[:, :Hq * D], buf[:, Hq * D:(Hq + Hk) * D], buf[:, (Hq + Hk) * D:]
        ops.qk_norm_rope_cache(q, k, v, qn, kn, pos, inv, slots, k_pool, v_pool, Hq, Hk, D, 1e-6, interleaved)

    run(qkv, kp, vp)
    with ops.force_reference():
        run(qkv2, kp2, vp2)
    _close(qkv[:, :Hq * D], qkv2[:, :Hq * D], rtol=2e-2, atol=5e-3)
    _close(kp, kp2, rtol=2e-2, atol=5e-3)
    assert torch.equal(vp, vp2)


def _paged_setup(B, ctxs, block_size, n_blocks):
    perm = torch.randperm(n_blocks, device=DEV).to(torch.int32)
    maxb = max((c + block_size - 1) // block_size for c in ctxs)
    bt = torch.zeros(B, maxb, dtype=torch.int32, device=DEV)
    used = 0
    for b, c in enumerate(ctxs):
        nb = (c + block_size - 1) // block_size
        bt[b, :nb] = perm[used:used + nb]
        used += nb
    return bt, torch.tensor(ctxs, dtype=torch.int32, device=DEV)


@pytest.mark.parametrize("Hq,Hkv,D", [(32, 8, 128), (4, 4, 64), (32, 4, 128), (8, 1, 256)])
@pytest.mark.parametrize("ctxs", [[1], [63, 64, 65], [700, 3, 129, 1024]])
def test_paged_decode_gqa(Hq, Hkv, D, ctxs):
    torch.manual_seed(0)
    B, bs = len(ctxs), 16
    bt, cl = _paged_setup(B, ctxs, bs, 256)
    kp, vp = _bf(256 * bs, Hkv, D), _bf(256 * bs, Hkv, D)
    q = _bf(B, Hq, D)
    scale = D ** -0.5
    for splits in (1, 3):
        o = ops.paged_attention(q, kp, vp, bt, cl, Hq=Hq, Hkv=Hkv, dqk=D, dv=D, block_size=bs, scale=scale, splits=splits)
        with ops.force_reference():
            o_ref = ops.paged_attention(q, kp, vp, bt, cl, Hq=Hq, Hkv=Hkv, dqk=D, dv=D, block_size=bs, scale=scale)
        _close(o, o_ref, rtol=2e-2, atol=1e-2)


def test_paged_decode_sliding_window():
    Hq, Hkv, D, bs = 8, 2, 128, 16
    ctxs = [300, 40]
    bt, cl = _paged_setup(2, ctxs, bs, 64)
    kp, vp, q = _bf(64 * bs, Hkv, D), _bf(64 * bs, Hkv, D), _bf(2, Hq, D)
    o = ops.paged_attention(q, kp, vp, bt, cl, Hq=Hq, Hkv=Hkv, dqk=D, dv=D, block_size=bs, scale=D ** -0.5, window=100, splits=2)
    with ops.force_reference():
        o_ref = ops.paged_attention(q, kp, vp, bt, cl, Hq=Hq, Hkv=Hkv, dqk=D, dv=D, block_size=bs, scale=D ** -0.5, window=100)
    _close(o, o_ref, rtol=2e-2, atol=1e-2)


@pytest.mark.parametrize("H,R,dr,dvo,ctxs", [(20, 512, 64, 256, [1, 100, 4096]), (4, 64, 32, 32, [5, 77, 200]),
                                             (20, 512, 64, 256, [2049] * 9)])
def test_mla_decode_with_value_up_projection(H, R, dr, dvo, ctxs):
    torch.manual_seed(1)
    B, bs = len(ctxs), 16
    n_blocks = sum((c + bs - 1) // bs for c in ctxs) + 4
    bt, cl = _paged_setup(B, ctxs, bs, n_blocks)
    cache = _bf(n_blocks * bs, R + dr, scale=0.5)
    q = _bf(B, H, R + dr, scale=0.3)
    w_uv = _bf(H, dvo, R, scale=0.05)
    scale = 1.0 / math.sqrt(192 + 64)
    o = ops.paged_attention(q, cache, None, bt, cl, Hq=H, Hkv=1, dqk=R + dr, dv=R, block_size=bs, scale=scale, w_uv=w_uv)
    with ops.force_reference():
        o_ref = ops.paged_attention(q, cache, None, bt, cl, Hq=H, Hkv=1, dqk=R + dr, dv=R, block_size=bs, scale=scale, w_uv=w_uv)
    _close(o, o_ref, rtol=3e-2, atol=1e-2)


@pytest.mark.parametrize("window", [0, 300])
def test_mla_decode_two_ctas_per_sm_variant(window):
    """More (sequence, split) CTAs than SMs: the launcher takes the 32-token-tile kernel with compact query rows."""
    torch.manual_seed(7)
    H, R, dr, dvo, bs = 20, 512, 64, 256, 16
    ctxs = [1, 31, 32, 33, 65, 700, 1000, 4096] * 3                     # 24 sequences
    B = len(ctxs)
    n_blocks = sum((c + bs - 1) // bs for c in ctxs) + 4
    bt, cl = _paged_setup(B, ctxs, bs, n_blocks)
    cache = _bf(n_blocks * bs, R + dr, scale=0.5)
    q = _bf(B, H, R + dr, scale=0.3)
    w_uv = _bf(H, dvo, R, scale=0.05)
    scale = 1.0 / math.sqrt(192 + 64)
    for splits in (7, 12):                                               # 168 and 288 CTAs
        o = ops.paged_attention(q, cache, None, bt, cl, Hq=H, Hkv=1, dqk=R + dr, dv=R, block_size=bs, scale=scale, w_uv=w_uv,
                                splits=splits, window=window)
        with ops.force_reference():
            o_ref = ops.paged_attention(q, cache, None, bt, cl, Hq=H, Hkv=1, dqk=R + dr, dv=R, block_size=bs, scale=scale, w_uv=w_uv,
                                        window=window)
        _close(o, o_ref, rtol=3e-2, atol=1e-2)
    assert ops.default_splits(32, 1, 4096, mla_latent=True) == 9 and ops.default_splits(1, 1, 4096, mla_latent=True) == 64


@pytest.mark.parametrize("T", [1, 5, 11])
def test_mla_prep(T):
    H, dn, dr, R = 20, 192, 64, 512
    q, kva = _bf(T, H * (dn + dr)), _bf(T, R + dr)
    w_ukT = _bf(H, R, dn, scale=0.05)
    nw = (1 + 0.1 * torch.randn(R, device=DEV)).to(torch.bfloat16)
    pos = torch.arange(100, 100 + T, dtype=torch.int32, device=DEV)
    inv = 1.0 / (1e6 ** (torch.arange(0, dr, 2, device=DEV).float() / dr))
    slots = torch.arange(T, device=DEV) * 2
    slots[-1] = -1 if T > 1 else 0
    qf1, qf2 = torch.zeros(T, H, R + dr, device=DEV, dtype=torch.bfloat16), torch.zeros(T, H, R + dr, device=DEV, dtype=torch.bfloat16)
    c1, c2 = torch.zeros(64, R + dr, device=DEV, dtype=torch.bfloat16), torch.zeros(64, R + dr, device=DEV, dtype=torch.bfloat16)
    ops.mla_prep(q, kva, w_ukT, nw, pos, inv, slots, qf1, c1, H, dn, dr, R, 1e-5, 1.0, True)
    with ops.force_reference():
        ops.mla_prep(q, kva, w_ukT, nw, pos, inv, slots, qf2, c2, H, dn, dr, R, 1e-5, 1.0, True)
    _close(qf1, qf2, rtol=2e-2, atol=5e-3)
    _close(c1, c2, rtol=2e-2, atol=5e-3)


@pytest.mark.parametrize("scoring,E,topk,ng,tg", [(0, 64, 4, 1, 1), (1, 64, 4, 1, 1), (1, 64, 8, 8, 4), (0, 128, 8, 1, 1),
                                                  (1, 8, 2, 1, 1)])
@pytest.mark.parametrize("T", [6, 200])      # 200 tokens: gate logits from the tensor-core GEMM + select kernel
def test_moe_router(scoring, E, topk, ng, tg, T):
    torch.manual_seed(3)
    K = 512
    x, d, w = _bf(T, K), _bf(T, K, scale=0.2), _bf(E, K, scale=0.2)
    nw = (1 + 0.1 * torch.randn(K, device=DEV)).to(torch.bfloat16)
    bias = torch.randn(E, device=DEV) * 0.1 if scoring == 1 else None
    r1, r2 = torch.empty_like(x), torch.empty_like(x)
    counts = torch.zeros(E, dtype=torch.int32, device=DEV)
    lg = torch.empty(T, E, device=DEV)
    ids, wts = ops.moe_router(x, w, delta=d, norm_w=nw, eps=1e-5, resid_out=r1, bias=bias, topk=topk, scoring=scoring,
                              renorm=True, routed_scale=1.8, n_group=ng, topk_group=tg, logits_out=lg, counts=counts)
    with ops.force_reference():
        ids_ref, wts_ref = ops.moe_router(x, w, delta=d, norm_w=nw, eps=1e-5, resid_out=r2, bias=bias, topk=topk,
                                          scoring=scoring, renorm=True, routed_scale=1.8, n_group=ng, topk_group=tg)
    assert torch.equal(r1, r2)
    # near-ties may order differently: compare as sets with their weights
    for t in range(T):
        a = dict(zip(ids[t].tolist(), wts[t].tolist()))
        b = dict(zip(ids_ref[t].tolist(), wts_ref[t].tolist()))
        common = set(a) & set(b)
        assert len(common) >= topk - 1
        for e in common:
            assert abs(a[e] - b[e]) < 2e-2 * max(1.0, abs(b[e]))
    assert int(counts.sum()) == T * topk


def test_argmax_and_greedy_sampler():
    lg = torch.randn(5, 154880, device=DEV)
    assert torch.equal(ops.argmax(lg), lg.argmax(-1))
    t = torch.zeros(5, device=DEV)
    assert torch.equal(ops.sample(lg, temperature=t), lg.argmax(-1))


def test_sampler_topk_topp_support_and_distribution():
    torch.manual_seed(0)
    V = 4096
    lg = torch.randn(1, V, device=DEV) * 2
    B = 512
    rows = lg.expand(B, V).contiguous()
    temp = torch.full((B,), 0.8, device=DEV)
    topk = torch.full((B,), 8, dtype=torch.int32, device=DEV)
    topp = torch.full((B,), 0.9, device=DEV)
    ids = ops.sample(rows, temperature=temp, top_k=topk, top_p=topp, seed=7, offset=0)
    # support: inside the top-8, and inside the 0.9 nucleus of the renormalised top-8
    sv, si = torch.sort(lg[0] / 0.8, descending=True)
    p = torch.softmax(sv[:8], -1)
    n_keep = int((p.cumsum(-1) < 0.9).sum()) + 1
    allowed = set(si[:n_keep].tolist())
    assert set(ids.tolist()) <= allowed
    # distribution: empirical frequency of the most likely token close to its renormalised probability
    pk = torch.softmax(sv[:n_keep], -1)
    freq = float((ids == si[0]).float().mean())
    assert abs(freq - float(pk[0])) < 0.08
    # different seeds give different draws; the same seed repeats
    a = ops.sample(rows, temperature=temp, top_k=topk, top_p=topp, seed=7, offset=0)
    b = ops.sample(rows, temperature=temp, top_k=topk, top_p=topp, seed=8, offset=0)
    assert torch.equal(a, ids) and not torch.equal(b, ids)


def test_sampler_gumbel_full_vocab_distribution():
    V, B = 64, 4096
    lg = torch.randn(1, V, device=DEV)
    rows = lg.expand(B, V).contiguous()
    ids = ops.sample(rows, temperature=torch.ones(B, device=DEV), seed=3)
    emp = torch.bincount(ids, minlength=V).float() / B
    assert float((emp - torch.softmax(lg[0], -1)).abs().max()) < 0.04


def test_sampler_repetition_penalty():
    V = 1000
    lg = torch.zeros(1, V, device=DEV)
    lg[0, 10] = 5.0
    lg[0, 20] = 4.0
    hist = torch.tensor([[10, -1, -1]], device=DEV)
    out = ops.sample(lg, temperature=torch.zeros(1, device=DEV), history=hist, rep_penalty=torch.tensor([2.0], device=DEV))
    assert int(out[0]) == 20
