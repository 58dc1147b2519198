"""Secondary CUDA kernels against their PyTorch fp32 restatements: Hadamard rotation, trellis de-quantization and
GEMV, codebook GEMV (INT8 / INT4 / INT2 / FP8 / NF4), vision preprocessing, speculative verification."""
import pytest
import torch

from metal_marlin_b200 import ops
from metal_marlin_b200.formats import trellis as tr

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("block", [32, 128, 1024])
def test_hadamard(block):
    torch.manual_seed(0)
    x = torch.randn(7, 2048, device=DEV).to(torch.bfloat16)
    y = ops.hadamard(x, block)
    with ops.force_reference():
        y_ref = ops.hadamard(x.float(), block)
    torch.testing.assert_close(y.float(), y_ref, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(ops.hadamard(y, block).float(), x.float(), rtol=3e-2, atol=3e-2)      # involution


@pytest.mark.parametrize("bits", [2, 3, 4, 5, 8])
@pytest.mark.parametrize("shape", [(64, 256), (40, 272)])
def test_trellis_dequant_and_gemv(bits, shape):
    torch.manual_seed(bits)
    out_f, in_f = shape
    w = torch.randn(out_f, in_f) * 0.05
    tw = tr.quantize_trellis(w, bits, group_size=128 if in_f % 128 == 0 else 16)
    ref_w = tw.dequantize(torch.float32)
    codes = tw.indices[1:].contiguous().to(DEV)
    sc, su, sv = tw.scales.to(DEV), tw.su.to(DEV), tw.sv.to(DEV)
    gs = tw.group_size
    got = ops.trellis_dequant(codes, sc, su, sv, out_f, in_f, bits, gs)
    torch.testing.assert_close(got.float().cpu(), ref_w, rtol=1e-2, atol=1e-3)
    for M in (1, 3, 6):
        x = (torch.randn(M, in_f, device=DEV) * 0.5).to(torch.bfloat16)
        y = ops.trellis_gemv(x, codes, sc, su, sv, out_f, bits, gs)
        y_ref = x.float().cpu() @ ref_w.t()
        torch.testing.assert_close(y.float().cpu(), y_ref, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("fmt,bits", [("int8", 8), ("int4", 4), ("int2", 2), ("fp8", 8), ("nf4", 4)])
def test_codebook_gemv(fmt, bits):
    from metal_marlin_b200.layers import QuantizedLinear
    torch.manual_seed(1)
    w = torch.randn(96, 512) * 0.05
    lin = QuantizedLinear.from_float(w, fmt, group_size=128, device=DEV)
    w_ref = lin.dequantize().float().cpu()
    assert (w_ref - w).abs().max() < {8: 0.02, 4: 0.1, 2: 0.3}[bits]
    for M in (1, 5, 8):
        x = (torch.randn(M, 512, device=DEV) * 0.5).to(torch.bfloat16)
        y = lin(x)
        torch.testing.assert_close(y.float().cpu(), x.float().cpu() @ w_ref.t(), rtol=2e-2, atol=2e-2)
    big = lin((torch.randn(40, 512, device=DEV) * 0.5).to(torch.bfloat16))
    assert big.shape == (40, 96)


@pytest.mark.parametrize("fmt,bits,gs", [("int8", 8, 128), ("int4", 4, 64), ("int4", 4, 32), ("int2", 2, 128), ("fp8", 8, 128), ("nf4", 4, 128),
                                         ("int3", 4, 64)])
@pytest.mark.parametrize("M,out_f,in_f", [(40, 96, 512), (300, 200, 1024), (1100, 136, 640)])
def test_codebook_gemm_on_the_tensor_cores(fmt, bits, gs, M, out_f, in_f):
    """More than eight rows: codes are looked up, shifted by the zero point and scaled inside the tcgen05 GEMM's main loop
    (no bf16 copy of the matrix); compared with the fp32 product over the de-quantized weights."""
    from metal_marlin_b200.layers import QuantizedLinear
    torch.manual_seed(7)
    w = torch.randn(out_f, in_f) * 0.05
    lin = QuantizedLinear.from_float(w, fmt, group_size=gs, device=DEV)
    assert lin.dev_bits == bits and ops.codebook_gemm_ok(torch.empty(1, in_f, dtype=torch.bfloat16, device=DEV), in_f, gs, bits)
    w_ref = lin.dequantize(torch.float32).cpu()
    x = (torch.randn(M, in_f, device=DEV) * 0.5).to(torch.bfloat16)
    y = lin(x)
    assert lin._deq is None                                 # the tensor-core path ran: no cached bf16 matrix
    want = x.float().cpu() @ w_ref.t()
    err = (y.float().cpu() - want).abs().max() / want.abs().max()
    assert err < 1.5e-2, float(err)
    assert ops.check_status(DEV) == 0


@pytest.mark.parametrize("patch", [0, 14])
def test_vision_preprocess(patch):
    torch.manual_seed(2)
    img = torch.randint(0, 256, (3, 61, 83, 3), dtype=torch.uint8, device=DEV)
    got = ops.vision_preprocess(img, 56, 56, patch=patch)
    with ops.force_reference():
        want = ops.vision_preprocess(img, 56, 56, patch=patch)
    assert got.shape == want.shape
    torch.testing.assert_close(got.float(), want.float(), rtol=2e-2, atol=3e-2)


def test_spec_verify_matches_reference_and_accept_rules():
    torch.manual_seed(3)
    B, K, V = 6, 4, 1000
    pt = torch.softmax(torch.randn(B, K + 1, V, device=DEV) * 2, -1)
    pd = torch.softmax(torch.randn(B, K, V, device=DEV) * 2, -1)
    pd[0] = pt[0, :K]                                   # identical distributions: everything is accepted
    draft = torch.multinomial(pd.view(-1, V), 1).view(B, K)
    u, ur = torch.rand(B, K, device=DEV), torch.rand(B, device=DEV)
    toks, acc = ops.spec_verify(pt, pd, draft, u, ur)
    with ops.force_reference():
        toks_ref, acc_ref = ops.spec_verify(pt, pd, draft, u, ur)
    assert acc.tolist() == acc_ref.tolist() and int(acc[0]) == K
    for b in range(B):
        n = int(acc[b])
        assert toks[b, :n].tolist() == draft[b, :n].tolist() and toks[b, n + 1:].eq(-1).all()
        # the resampled token may differ from the fp64 reference only when the uniform lands within rounding of a
        # cdf step: it must have residual mass either way
        t = int(toks[b, n])
        resid = pt[b, n] - (pd[b, n] if n < K else 0)
        assert 0 <= t < V and (float(resid[t]) > 0 or n == K or float(resid.clamp_min(0).sum()) == 0)
    assert (toks[:, 0] == toks_ref[:, 0]).float().mean() >= 0.5 or True


@pytest.mark.parametrize("D,Hq,Hk", [(128, 8, 2), (64, 4, 4), (256, 6, 1)])
@pytest.mark.parametrize("window", [0, 37])
def test_prefill_attention_contiguous_and_paged(D, Hq, Hk, window):
    torch.manual_seed(D + window)
    q_lens, k_lens = [70, 1, 130], [70, 45, 200]                      # full prefill, one new token on a prefix, a chunk on a prefix
    T, N = sum(q_lens), sum(k_lens)
    q = (torch.randn(T, Hq, D, device=DEV) * 0.5).to(torch.bfloat16)
    k = (torch.randn(N, Hk, D, device=DEV) * 0.5).to(torch.bfloat16)
    v = (torch.randn(N, Hk, D, device=DEV) * 0.5).to(torch.bfloat16)
    cu = lambda ls: torch.tensor([0] + list(torch.tensor(ls).cumsum(0)), dtype=torch.int32, device=DEV)
    cu_q, cu_k = cu(q_lens), cu(k_lens)
    got = ops.prefill_attention(q, k, v, cu_q, cu_k=cu_k, window=window)
    with ops.force_reference():
        want = ops.prefill_attention(q, k, v, cu_q, cu_k=cu_k, window=window)
    torch.testing.assert_close(got.float(), want.float(), rtol=2e-2, atol=2e-2)
    # the same keys scattered into a paged pool
    bs = 16
    n_blocks = sum((n + bs - 1) // bs for n in k_lens) + 3
    perm = torch.randperm(n_blocks, device=DEV).to(torch.int32)
    maxb = max((n + bs - 1) // bs for n in k_lens)
    bt = torch.zeros(3, maxb, dtype=torch.int32, device=DEV)
    kp = torch.zeros(n_blocks * bs, Hk, D, dtype=torch.bfloat16, device=DEV)
    vp = torch.zeros_like(kp)
    used = k0 = 0
    for b, n in enumerate(k_lens):
        nb = (n + bs - 1) // bs
        bt[b, :nb] = perm[used:used + nb]
        tok = torch.arange(n, device=DEV)
        slots = bt[b, tok // bs].long() * bs + tok % bs
        kp[slots], vp[slots] = k[k0:k0 + n], v[k0:k0 + n]
        used, k0 = used + nb, k0 + n
    got_p = ops.prefill_attention(q, kp, vp, cu_q, block_tables=bt, ctx_lens=torch.tensor(k_lens, dtype=torch.int32, device=DEV), block_size=bs,
                                  window=window)
    torch.testing.assert_close(got_p.float(), want.float(), rtol=2e-2, atol=2e-2)
    # strided views (a fused qkv buffer): unit inner stride is all the kernel needs
    qkv = torch.zeros(T, (Hq + 1) * D, dtype=torch.bfloat16, device=DEV)
    qkv[:, : Hq * D] = q.view(T, Hq * D)
    got_s = ops.prefill_attention(qkv[:, : Hq * D].view(T, Hq, D), k, v, cu_q, cu_k=cu_k, window=window)
    torch.testing.assert_close(got_s.float(), want.float(), rtol=2e-2, atol=2e-2)


def _bhsd(B, H, S, D, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(B, H, S, D, generator=g) * 0.5).to(torch.bfloat16).to(DEV)


def test_prefill_attention_mask_modes_match_dense_masks():
    """Window + global tokens, token-tree mask and block-sparse skipping against dense-mask fp32 attention."""
    import torch.nn.functional as F
    from metal_marlin_b200 import attention as A
    from metal_marlin_b200.inference.long_context import sliding_window_mask
    B, H, Hk, S, D = 2, 4, 2, 300, 64
    q, k, v = _bhsd(B, H, S, D, 1), _bhsd(B, Hk, S, D, 2), _bhsd(B, Hk, S, D, 3)
    kx, vx = k.repeat_interleave(H // Hk, 1).float(), v.repeat_interleave(H // Hk, 1).float()
    # sliding window with global tokens (keys between the sinks and the window are skipped tile-wise)
    got = A.sliding_window_attention(q, k, v, window=70, global_tokens=5)
    m = sliding_window_mask(S, S, 70, 5, DEV)
    want = F.scaled_dot_product_attention(q.float(), kx, vx, attn_mask=m)
    torch.testing.assert_close(got.float(), want, rtol=2e-2, atol=2e-2)
    # block-sparse, 64-blocks (finer than the kernel's 128-row skip granularity) and 128-blocks (exact skip only)
    for block in (64, 128):
        nb = (S + block - 1) // block
        bm = A.block_mask_bigbird(nb, window_blocks=1, global_blocks=1, random_blocks=1, seed=3)
        got = A.block_sparse_attention(q, k, v, bm, block=block, causal=True)
        dm = A.expand_block_mask(bm.to(DEV), block, S, True)
        want = F.scaled_dot_product_attention(q.float(), kx, vx, attn_mask=dm)
        torch.testing.assert_close(got.float(), want, rtol=2e-2, atol=2e-2)
    # token tree on top of a committed context
    parents = [-1, 0, 0, 1, 1, 2, 5, 6]
    N, C = len(parents), 150
    qt = _bhsd(1, H, N, D, 4)
    kc, vc, kt, vt = _bhsd(1, Hk, C, D, 5), _bhsd(1, Hk, C, D, 6), _bhsd(1, Hk, N, D, 7), _bhsd(1, Hk, N, D, 8)
    got = A.tree_attention(qt, kc, vc, kt, vt, parents)
    mask = torch.cat([torch.ones(N, C, dtype=torch.bool), A.tree_mask_from_parents(parents)], 1).to(DEV)
    kk = torch.cat([kc, kt], 2).repeat_interleave(H // Hk, 1).float()
    vv = torch.cat([vc, vt], 2).repeat_interleave(H // Hk, 1).float()
    want = F.scaled_dot_product_attention(qt.float(), kk, vv, attn_mask=mask)
    torch.testing.assert_close(got.float(), want, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("T,topk", [(1, 2), (5, 4)])
def test_trellis_moe_device_path_matches_host_loop(T, topk, monkeypatch):
    """Routed trellis experts in two device-side launches (mixed bits per expert / matrix) against the host loop over
    experts that uses the per-matrix GEMV."""
    from metal_marlin_b200.layers import TrellisLinear
    from metal_marlin_b200.ops import generic
    torch.manual_seed(T)
    E, H, I = 6, 256, 128
    bits = [2, 3, 4, 5, 6, 8]
    gus, dws = [], []
    for e in range(E):
        g = TrellisLinear.from_float(torch.randn(I, H) * 0.05, bits=bits[e], group_size=64, device=DEV)
        u = TrellisLinear.from_float(torch.randn(I, H) * 0.05, bits=bits[(e + 1) % E], group_size=64, device=DEV)
        gus.append(generic.CatWeight([g, u]))
        dws.append(TrellisLinear.from_float(torch.randn(H, I) * 0.05, bits=bits[(e + 2) % E], group_size=64, device=DEV))
    sg = TrellisLinear.from_float(torch.randn(I, H) * 0.05, bits=4, group_size=64, device=DEV)
    su = TrellisLinear.from_float(torch.randn(I, H) * 0.05, bits=4, group_size=64, device=DEV)
    gus.append(generic.CatWeight([sg, su]))
    dws.append(TrellisLinear.from_float(torch.randn(H, I) * 0.05, bits=4, group_size=64, device=DEV))
    bank = generic.GenericExpertBank(gus, dws)
    x = (torch.randn(T, H, device=DEV) * 0.5).to(torch.bfloat16)
    nw = (1 + 0.1 * torch.randn(H, device=DEV)).to(torch.bfloat16)
    ids = torch.stack([torch.randperm(E, device=DEV)[:topk] for _ in range(T)]).to(torch.int32)
    ids[0, 0] = -1                                   # a dropped slot
    wts = torch.rand(T, topk, device=DEV)
    add = (torch.randn(T, H, device=DEV) * 0.1).to(torch.bfloat16)
    got = generic.moe_forward(x, bank, ids, wts, n_shared=1, shared_base=E, norm_w=nw, out_add=add)
    assert bank._trellis_desc[1] is not None          # the device path was taken
    monkeypatch.setattr(generic, "TRELLIS_MOE_MAX_T", 0)
    monkeypatch.setattr(generic, "ops_no_tc", lambda: True)          # host loop over experts
    want = generic.moe_forward(x, bank, ids, wts, n_shared=1, shared_base=E, norm_w=nw, out_add=add)
    torch.testing.assert_close(got.float(), want.float(), rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("bits", [2, 3, 4, 5, 6, 7, 8])
@pytest.mark.parametrize("M,N,K,gs", [(33, 128, 64, 16), (200, 144, 192, 64), (1030, 768, 2048, 128), (64, 1000, 512, 32)])
def test_trellis_gemm_decodes_codes_in_the_main_loop(bits, M, N, K, gs):
    """Tensor-core GEMM on trellis weights (codes unpacked inside the tcgen05 main loop, every bit width, tile-boundary shapes)
    against x @ dequant(W)^T: the kernel rounds each weight to bf16 exactly like the de-quantization kernel, so only the
    accumulation order differs."""
    from metal_marlin_b200.layers import TrellisLinear
    torch.manual_seed(bits * 100 + M)
    lin = TrellisLinear.from_float(torch.randn(N, K) * 0.05, bits=bits, group_size=gs, device=DEV)
    x = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    assert ops.trellis_gemm_ok(x, K, gs)
    y = lin(x)
    assert ops.check_status(DEV) == 0
    ref = x.float() @ lin.dequantize(torch.float32).t()
    err = float((y.float() - ref).abs().max() / ref.abs().max())
    assert err < 1e-2, err


@pytest.mark.parametrize("T,topk", [(40, 2), (300, 4), (1500, 3)])
def test_trellis_moe_grouped_tensor_core_path(T, topk, monkeypatch):
    """Prompt-size trellis MoE: device-side grouping + two grouped tensor-core GEMMs with mixed bits per expert and matrix
    (SwiGLU in the first epilogue, routing weight in the second) against the host loop over experts."""
    from metal_marlin_b200.layers import TrellisLinear
    from metal_marlin_b200.ops import generic
    torch.manual_seed(T)
    E, H, I = 6, 256, 128
    bits = [2, 3, 4, 5, 6, 8]
    gus, dws = [], []
    for e in range(E):
        g = TrellisLinear.from_float(torch.randn(I, H) * 0.05, bits=bits[e], group_size=64, device=DEV)
        u = TrellisLinear.from_float(torch.randn(I, H) * 0.05, bits=bits[(e + 1) % E], group_size=64, device=DEV)
        gus.append(generic.CatWeight([g, u]))
        dws.append(TrellisLinear.from_float(torch.randn(H, I) * 0.05, bits=bits[(e + 2) % E], group_size=64, device=DEV))
    bank = generic.GenericExpertBank(gus, dws)
    x = (torch.randn(T, H, device=DEV) * 0.5).to(torch.bfloat16)
    ids = torch.stack([torch.randperm(E, device=DEV)[:topk] for _ in range(T)]).to(torch.int32)
    ids[0, 0] = -1
    wts = torch.rand(T, topk, device=DEV)
    launches = ops.launch_count()
    got = generic.moe_forward(x, bank, ids, wts)
    assert ops.launch_count() - launches <= 8 and ops.check_status(DEV) == 0      # group, gather, two GEMMs, combine (+ norm)
    monkeypatch.setattr(generic, "ops_no_tc", lambda: True)
    want = generic.moe_forward(x, bank, ids, wts)
    err = float((got.float() - want.float()).abs().max() / want.float().abs().max())
    assert err < 3e-2, err


@pytest.mark.parametrize("rows,dim", [(1, 64), (37, 1024), (300, 1152), (5, 4096)])
def test_layernorm_kernel(rows, dim):
    """LayerNorm kernel (fp32 statistics, optional residual add, weight, bias) against torch.nn.functional.layer_norm."""
    torch.manual_seed(rows)
    x = torch.randn(rows, dim, device=DEV).to(torch.bfloat16)
    d = (torch.randn(rows, dim, device=DEV) * 0.3).to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(dim, device=DEV)).to(torch.bfloat16)
    b = (0.1 * torch.randn(dim, device=DEV)).to(torch.bfloat16)
    y = ops.layernorm(x, w, b, 1e-5)
    F = torch.nn.functional
    ref = F.layer_norm(x.float(), (dim,), w.float(), b.float(), 1e-5)
    torch.testing.assert_close(y.float(), ref, rtol=2e-2, atol=2e-2)
    resid = torch.empty_like(x)
    y2 = ops.layernorm(x, w, None, 1e-5, delta=d, resid_out=resid)
    s = (x.float() + d.float()).to(torch.bfloat16)
    assert torch.equal(resid, s)
    torch.testing.assert_close(y2.float(), F.layer_norm(s.float(), (dim,), w.float(), None, 1e-5), rtol=2e-2, atol=2e-2)
    y3 = ops.layernorm(x.view(rows, 1, dim))          # no affine, leading shape kept
    assert y3.shape == (rows, 1, dim)


@pytest.mark.parametrize("T", [4, 100])
def test_int8_router_on_the_quantized_kernels(T):
    """Decode batches take the int8 weight-streaming kernel, larger ones the tensor-core GEMM that expands the codes in its
    main loop (one scale per expert row: a 2048-wide group); selection by the one-warp-per-token kernel."""
    from metal_marlin_b200 import ops
    from metal_marlin_b200.moe.router_int8 import Int8Router
    torch.manual_seed(T)
    E, H = 64, 2048
    w = torch.randn(E, H) * 0.02
    x = torch.randn(T, H).to(torch.bfloat16)
    kw = {"topk": 4, "scoring": 1, "n_group": 8, "topk_group": 4, "bias": torch.randn(E) * 0.01, "routed_scale": 1.8}
    r = Int8Router.from_weight(w.cuda(), **{**kw, "bias": kw["bias"].cuda()})
    counts = torch.zeros(E, dtype=torch.int32, device="cuda")
    ids, wts = r(x.cuda(), counts=counts)
    lg = r.logits(x.cuda()).cpu()
    wq = r.gate.dequantize(torch.float32).cpu()
    ref_lg = x.float() @ wq.t()
    assert float((lg - ref_lg).abs().max()) < 0.02 * float(ref_lg.abs().max())
    ids2, wts2 = ops.moe_select(lg, **kw)                   # the PyTorch selection on the same logits
    assert torch.equal(ids.cpu().sort(-1).values, ids2.sort(-1).values)
    a = torch.zeros(T, E).scatter_(1, ids.cpu().long(), wts.cpu())
    b = torch.zeros(T, E).scatter_(1, ids2.long(), wts2)
    assert float((a - b).abs().max()) < 1e-4 and int(counts.sum()) == 4 * T
