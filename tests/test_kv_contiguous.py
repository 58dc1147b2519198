"""Contiguous KV caches: storage modes, sliding eviction, snapshot / restore, MLA latent growth, prefix reuse.
Modelled on the reference's tests/test_kv_cache*.py and test_mla_kv_cache.py."""
import pytest
import torch

from metal_marlin_b200.kv.contiguous import (CacheConfig, KVCache, MLAKVCache, PersistentKVCache, dequantize_kv, quantize_kv)


@pytest.mark.parametrize("mode,tol", [("bf16", 1e-2), ("fp16", 1e-3), ("fp8", 0.07), ("fp8_e5m2", 0.15), ("int8", 0.02), ("fp4", 0.3)])
def test_quantize_roundtrip(mode, tol):
    torch.manual_seed(0)
    x = torch.randn(2, 3, 5, 64)
    st, sc = quantize_kv(x, mode)
    y = dequantize_kv(st, sc, mode, torch.float32)
    assert y.shape == x.shape
    assert (y - x).abs().max() / x.abs().max() < tol
    if mode == "fp4":
        assert st.dtype == torch.uint8 and st.shape[-1] == 32


@pytest.mark.parametrize("layout", ["BHSD", "BSHD"])
@pytest.mark.parametrize("mode", ["bf16", "fp8", "int8"])
def test_kv_cache_update_and_positions(layout, mode):
    cfg = CacheConfig(num_layers=2, num_kv_heads=2, head_dim=16, max_seq_len=32, dtype=mode, layout=layout)
    c = KVCache(cfg)
    torch.manual_seed(1)
    shape = (lambda T: (1, 2, T, 16)) if layout == "BHSD" else (lambda T: (1, T, 2, 16))
    ks = [torch.randn(*shape(5)), torch.randn(*shape(1))]
    for k in ks:
        for layer in range(2):
            ka, va = c.update(layer, k, k * 2, dtype=torch.float32)
    assert c.seq_len == 6
    full = torch.cat(ks, 2 if layout == "BHSD" else 1)
    assert (ka - full).abs().max() < 0.2 and (va - 2 * full).abs().max() < 0.4


def test_sliding_window_eviction_keeps_sinks():
    cfg = CacheConfig(num_layers=1, num_kv_heads=1, head_dim=8, max_seq_len=16, sliding_window=8, sink_tokens=2, dtype="fp16")
    c = KVCache(cfg)
    for i in range(12):
        k = torch.full((1, 1, 1, 8), float(i))
        ka, _ = c.update(0, k, k, dtype=torch.float32)
    assert c.seq_len == 8 and c.total_seen == 12
    assert ka[0, 0, :, 0].tolist() == [0.0, 1.0, 6.0, 7.0, 8.0, 9.0, 10.0, 11.0]
    full = KVCache(CacheConfig(num_layers=1, num_kv_heads=1, head_dim=8, max_seq_len=4))
    with pytest.raises(RuntimeError):
        full.update(0, torch.zeros(1, 1, 5, 8), torch.zeros(1, 1, 5, 8))


def test_snapshot_restore_and_truncate():
    c = KVCache(CacheConfig(num_layers=1, num_kv_heads=1, head_dim=4, max_seq_len=16, dtype="fp16"))
    c.update(0, torch.ones(1, 1, 3, 4), torch.ones(1, 1, 3, 4))
    snap = c.snapshot()
    c.update(0, torch.full((1, 1, 2, 4), 5.0), torch.full((1, 1, 2, 4), 5.0))
    assert c.seq_len == 5
    c.restore(snap)
    assert c.seq_len == 3 and float(c.get(0, torch.float32)[0].sum()) == 12.0
    c.truncate(1)
    assert c.seq_len == 1


@pytest.mark.parametrize("mode", ["bf16", "fp8", "fp4"])
def test_mla_cache_grows_and_snapshots(mode):
    c = MLAKVCache(num_layers=2, kv_lora_rank=64, rope_dim=16, max_seq_len=64, dtype=mode, initial_seq_len=4)
    torch.manual_seed(2)
    rows = torch.randn(1, 9, 80)
    for layer in range(2):
        out = c.update_compressed(layer, rows, dtype=torch.float32)
    assert c.seq_len == 9 and c.capacity >= 9 and out.shape == (1, 9, 80)
    assert (out - rows).abs().max() / rows.abs().max() < (0.3 if mode == "fp4" else 0.08)
    snap = c.snapshot()
    c.update_compressed(0, rows[:, :1]), c.update_compressed(1, rows[:, :1])
    c.restore(snap)
    assert c.seq_len == 9
    with pytest.raises(RuntimeError):
        c.update_compressed(0, torch.randn(1, 100, 80))


def test_persistent_prefix_reuse():
    c = KVCache(CacheConfig(num_layers=1, num_kv_heads=1, head_dim=4, max_seq_len=32, dtype="fp16"))
    p = PersistentKVCache(c)
    assert p.match([1, 2, 3, 4]) == 0
    c.update(0, torch.zeros(1, 1, 4, 4), torch.zeros(1, 1, 4, 4))
    p.extend([1, 2, 3, 4])
    assert p.match([1, 2, 3, 9, 9]) == 3 and c.seq_len == 3
    assert p.match([1, 2, 3]) == 2          # at least one token is left to prefill
