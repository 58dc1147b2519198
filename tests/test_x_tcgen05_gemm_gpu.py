"""tcgen05 / TMA / TMEM GEMM kernels against fp32 PyTorch matmuls (tile-boundary shapes, every token
tile, grouped MoE mode, batched bf16 mode).  Also asserts the bounded-wait status word stays 0."""
import pytest
import torch

from metal_marlin_b200 import ops
from metal_marlin_b200.ops import FP4ExpertBank, FP4Weight

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _check(y, ref, tol=2e-2):
    err = (y.float() - ref.float()).abs().max() / ref.float().abs().max().clamp_min(1e-6)
    assert float(err) < tol, float(err)


@pytest.mark.parametrize("M", [17, 32, 33, 64, 100, 128, 257, 1024, 2500])
@pytest.mark.parametrize("N,K,gs", [(128, 64, 64), (256, 512, 128), (2048, 2048, 128), (576, 768, 128), (1000, 1536, 128),
                                    (48, 192, 64)])
def test_fp4_gemm_tcgen05(M, N, K, gs):
    torch.manual_seed(M + N)
    W = FP4Weight.from_float(torch.randn(N, K, device=DEV) * 0.03, gs)
    x = (torch.randn(M, K, device=DEV)).to(torch.bfloat16)
    y = ops.linear(x, W)
    assert ops.check_status(DEV) == 0
    ref = x.float() @ W.dequantize().t()
    _check(y, ref)


def test_fp4_gemm_large_scale_values_use_two_step_rescale():
    N, K = 128, 256
    codes = torch.randint(0, 16, (N, K), dtype=torch.uint8, device=DEV)
    scales = torch.full((N, K // 128), 8.0, dtype=torch.float16, device=DEV)     # >= 2: no folding of 2^126
    W = FP4Weight.from_codes(codes, scales)
    x = torch.randint(-2, 3, (40, K), device=DEV).to(torch.bfloat16)
    y = ops.linear(x, W)
    _check(y, x.float() @ W.dequantize().t(), tol=1e-2)


@pytest.mark.parametrize("M,N,K", [(40, 128, 64), (300, 1000, 512), (128, 256, 2048)])
def test_bf16_gemm_tcgen05(M, N, K):
    x = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    w = torch.randn(N, K, device=DEV).to(torch.bfloat16)
    y = ops.bf16_gemm(x, w, out_dtype=torch.float32)
    assert ops.check_status(DEV) == 0
    _check(y, x.float() @ w.float().t(), tol=1e-2)


def test_bf16_gemm_batched_shared_x():
    x = torch.randn(70, 128, device=DEV).to(torch.bfloat16)
    w = torch.randn(5, 192, 128, device=DEV).to(torch.bfloat16)
    y = ops.bf16_gemm(x, w)
    _check(y, torch.einsum("mk,bnk->bmn", x.float(), w.float()), tol=1e-2)


@pytest.mark.parametrize("T,E,topk,ns", [(64, 8, 2, 1), (300, 64, 4, 1), (1000, 16, 8, 0)])
def test_moe_grouped_gemm_path(T, E, topk, ns, monkeypatch):
    torch.manual_seed(T)
    monkeypatch.setattr(ops, "MOE_GROUPED_GEMV_MAX_T", 0)      # 64 tokens would otherwise take the streaming kernel
    H, I = 256, 128
    gu = FP4ExpertBank.from_float(torch.randn(E + ns, 2 * I, H, device=DEV) * 0.05, 64)
    dn = FP4ExpertBank.from_float(torch.randn(E + ns, H, I, device=DEV) * 0.05, 64)
    x = torch.randn(T, H, device=DEV).to(torch.bfloat16)
    nw = (1 + 0.1 * torch.randn(H, device=DEV)).to(torch.bfloat16)
    ids = torch.stack([torch.randperm(E, device=DEV)[:topk] for _ in range(T)]).to(torch.int32)
    wts = torch.rand(T, topk, device=DEV)
    y = ops.moe_forward(x, gu, dn, ids, wts, n_shared=ns, shared_base=E, norm_w=nw)
    assert ops.check_status(DEV) == 0
    with ops.force_reference():
        y_ref = ops.moe_forward(x, gu, dn, ids, wts, n_shared=ns, shared_base=E, norm_w=nw)
    _check(y, y_ref, tol=4e-2)


@pytest.mark.parametrize("T,E,topk,ns,H,I,gs", [(17, 8, 2, 1, 256, 128, 64), (32, 64, 8, 1, 2048, 512, 128), (64, 16, 4, 0, 1024, 256, 32),
                                                (128, 32, 8, 2, 512, 192, 64), (40, 64, 6, 1, 2048, 1536, 128)])
def test_moe_grouped_streaming_path(T, E, topk, ns, H, I, gs):
    """17 to 128 tokens: tokens sorted by expert, 8-row tiles on the weight-streaming kernel (gather and routing
    weight fused)."""
    torch.manual_seed(T)
    gu = FP4ExpertBank.from_float(torch.randn(E + ns, 2 * I, H, device=DEV) * 0.05, gs)
    dn = FP4ExpertBank.from_float(torch.randn(E + ns, H, I, device=DEV) * 0.05, gs)
    x = torch.randn(T, H, device=DEV).to(torch.bfloat16)
    nw = (1 + 0.1 * torch.randn(H, device=DEV)).to(torch.bfloat16)
    # skewed routing: expert 0 gets far more than one tile of rows, some experts none
    ids = torch.stack([torch.randperm(E, device=DEV)[:topk] for _ in range(T)]).to(torch.int32)
    ids[: T // 2, 0] = 0
    ids[: T // 2, 1:] = torch.stack([1 + torch.randperm(E - 1, device=DEV)[: topk - 1] for _ in range(T // 2)]).to(torch.int32)
    wts = torch.rand(T, topk, device=DEV)
    add = torch.randn(T, H, device=DEV).to(torch.bfloat16)
    assert ops.MOE_GEMV_MAX_T < T <= ops.MOE_GROUPED_GEMV_MAX_T
    y = ops.moe_forward(x, gu, dn, ids, wts, n_shared=ns, shared_base=E, norm_w=nw, out_add=add)
    with ops.force_reference():
        y_ref = ops.moe_forward(x, gu, dn, ids, wts, n_shared=ns, shared_base=E, norm_w=nw, out_add=add)
    _check(y, y_ref, tol=4e-2)


def test_prefill_through_tensor_core_path_matches_reference():
    from metal_marlin_b200.models.mmfp4_causal_lm import MMFP4ForCausalLM, prefill
    lm = MMFP4ForCausalLM.from_config("tiny-mla-moe", device="cuda", seed=5)
    prompts = [torch.randint(0, 512, (200,)).tolist(), torch.randint(0, 512, (90,)).tolist()]
    bt = torch.arange(32, dtype=torch.int32).view(2, 16)
    a = prefill(lm.model, lm.new_cache(32, 16), prompts, bt)
    with ops.force_reference():
        b = prefill(lm.model, lm.new_cache(32, 16), prompts, bt)
    assert ops.check_status(DEV) == 0
    assert float((a - b).abs().max() / b.abs().max()) < 4e-2


@pytest.mark.parametrize("M", [33, 64, 130, 257, 1024, 2300])
@pytest.mark.parametrize("I,K,gs", [(64, 64, 64), (128, 512, 128), (1536, 2048, 128), (320, 768, 64)])
def test_fp4_gemm_swiglu_epilogue(M, I, K, gs):
    """SwiGLU fused into the tensor-core GEMM's epilogue (64 gate rows and the 64 matching up rows share one accumulator
    tile) against the fp32 statement silu(x Wg^T) * (x Wu^T)."""
    torch.manual_seed(M + I)
    W = FP4Weight.from_float(torch.randn(2 * I, K, device=DEV) * 0.05, gs)
    x = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    y = ops.linear(x, W, act=1)
    assert ops.check_status(DEV) == 0 and y.shape == (M, I)
    z = x.float() @ W.dequantize().t()
    ref = torch.nn.functional.silu(z[:, :I]) * z[:, I:]
    _check(y, ref, tol=3e-2)
    assert not torch.isnan(y.float()).any()


@pytest.mark.parametrize("T,E,topk,I", [(200, 8, 2, 128), (700, 16, 4, 192), (1500, 64, 4, 1536)])
def test_moe_grouped_gemm_swiglu_epilogue(T, E, topk, I, monkeypatch):
    """Grouped expert GEMM with the fused SwiGLU epilogue (ragged expert tiles) against the reference MoE."""
    torch.manual_seed(T)
    monkeypatch.setattr(ops, "MOE_GROUPED_GEMV_MAX_T", 0)
    H = 512
    gu = FP4ExpertBank.from_float(torch.randn(E, 2 * I, H, device=DEV) * 0.05, 64)
    dn = FP4ExpertBank.from_float(torch.randn(E, H, I, device=DEV) * 0.05, 64)
    x = torch.randn(T, H, device=DEV).to(torch.bfloat16)
    ids = torch.stack([torch.randperm(E, device=DEV)[:topk] for _ in range(T)]).to(torch.int32)
    wts = torch.rand(T, topk, device=DEV)
    y = ops.moe_forward(x, gu, dn, ids, wts)
    assert ops.check_status(DEV) == 0
    with ops.force_reference():
        y_ref = ops.moe_forward(x, gu, dn, ids, wts)
    _check(y, y_ref, tol=4e-2)
