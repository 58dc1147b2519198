"""Attention variants and long-context helpers against dense PyTorch references (reference:
tests/test_long_context.py, test_sliding_window*.py, test_tree_attention.py, test_diff_transformer.py)."""
import torch
import torch.nn.functional as F

from metal_marlin_b200 import attention as A
from metal_marlin_b200.inference.long_context import (LongContextConfig, StreamingAttention, chunked_attention, compress_kv,
                                                      sliding_window_mask)


def test_sliding_window_mask_and_chunked_attention_match_dense():
    torch.manual_seed(0)
    q, k, v = torch.randn(1, 4, 40, 16), torch.randn(1, 2, 40, 16), torch.randn(1, 2, 40, 16)
    m = sliding_window_mask(40, 40, window=8, global_tokens=2)
    assert m[39, 0] and m[39, 1] and not m[39, 2] and m[39, 32] and not m[39, 31] and not m[3, 4]
    ref = F.scaled_dot_product_attention(q, k.repeat_interleave(2, 1), v.repeat_interleave(2, 1), attn_mask=m)
    out = chunked_attention(q, k, v, chunk_size=16, window=8, global_tokens=2)
    torch.testing.assert_close(out, ref, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(A.sliding_window_attention(q, k, v, 8, 2), ref, rtol=1e-4, atol=1e-5)
    # decode-shaped: fewer queries than keys
    out2 = chunked_attention(q[:, :, -3:], k, v, chunk_size=16)
    ref2 = F.scaled_dot_product_attention(q, k.repeat_interleave(2, 1), v.repeat_interleave(2, 1), is_causal=True)[:, :, -3:]
    torch.testing.assert_close(out2, ref2, rtol=1e-4, atol=1e-5)


def test_kv_compression_and_streaming_bound_memory():
    cfg = LongContextConfig(global_tokens=2, compression_ratio=4, compression_threshold=16, sliding_window=8, chunk_size=8)
    k = torch.arange(40, dtype=torch.float32).view(1, 1, 40, 1).expand(1, 1, 40, 4).contiguous()
    kc, vc = compress_kv(k, k, cfg)
    assert kc.shape[2] == 2 + (40 - 16 - 2) // 4 + 16 + ((40 - 16 - 2) % 4)
    assert float(kc[0, 0, 2, 0]) == (2 + 3 + 4 + 5) / 4 and float(kc[0, 0, -1, 0]) == 39.0
    sa = StreamingAttention(cfg)
    for _ in range(30):
        o = sa(torch.randn(1, 1, 1, 4), torch.randn(1, 1, 1, 4), torch.randn(1, 1, 1, 4))
    assert sa.k.shape[2] == 10 and o.shape == (1, 1, 1, 4)


def test_block_sparse_masks():
    m = A.block_mask_sliding(6, 2)
    assert m[3, 2] and m[3, 3] and not m[3, 1] and not m[2, 3]
    bb = A.block_mask_bigbird(8, 2, global_blocks=1, random_blocks=1)
    assert bb[:, 0].all() and not bb[0, 1:].any()
    lf = A.block_mask_longformer(8, 2, (0, 4))
    assert lf[7, 4] and lf[7, 0] and not lf[7, 2]
    torch.manual_seed(1)
    q = torch.randn(1, 2, 24, 8)
    full = A.block_sparse_attention(q, q, q, torch.ones(6, 6, dtype=torch.bool), block=4)
    torch.testing.assert_close(full, F.scaled_dot_product_attention(q, q, q, is_causal=True), rtol=1e-4, atol=1e-5)


def test_tree_attention_matches_per_path_causal():
    torch.manual_seed(2)
    parents = [-1, 0, 0, 1, 2]                   # two branches under node 0
    m = A.tree_mask_from_parents(parents)
    assert m[3].tolist() == [True, True, False, True, False] and m[4].tolist() == [True, False, True, False, True]
    C, N, D = 6, 5, 8
    kc, vc = torch.randn(1, 1, C, D), torch.randn(1, 1, C, D)
    qt, kt, vt = torch.randn(1, 1, N, D), torch.randn(1, 1, N, D), torch.randn(1, 1, N, D)
    out = A.tree_attention(qt, kc, vc, kt, vt, parents)
    path = [0, 1, 3]                              # node 3 along its own path must equal plain causal attention
    k_path = torch.cat([kc, kt[:, :, path]], 2)
    v_path = torch.cat([vc, vt[:, :, path]], 2)
    ref = F.scaled_dot_product_attention(qt[:, :, 3:4], k_path, v_path)
    torch.testing.assert_close(out[:, :, 3:4], ref, rtol=1e-4, atol=1e-5)


def test_differential_attention_reduces_to_plain_when_lambda_zero():
    torch.manual_seed(3)
    q1, k1, q2, k2, v = (torch.randn(1, 2, 10, 8) for _ in range(5))
    o = A.differential_attention(q1, k1, q2, k2, v, lam=0.0, lambda_init=0.0)
    a = F.scaled_dot_product_attention(q1, k1, v, is_causal=True)
    torch.testing.assert_close(o, a * torch.rsqrt(a.pow(2).mean(-1, keepdim=True) + 1e-5), rtol=1e-4, atol=1e-5)
    assert abs(A.lambda_init_for_layer(0) - 0.2) < 1e-6
