"""Recycling buffer pool, transfer stream and ring buffer (``memory/pools.py``) on CPU.  Parity: reference
``tests/test_buffer_pool.py`` / ``tests/test_buffer_ring.py`` (reuse, best fit, eviction, idle cleanup, O(1) reset)."""
import torch

from metal_marlin_b200.memory import BufferPool, RingBuffer, TransferStream, get_ring_buffer, reset_ring_buffer


def test_buffer_pool_reuses_best_fit_and_evicts_lru():
    pool = BufferPool("cpu", max_bytes=4096, max_waste=2.0, idle_seconds=10.0)
    a, b = pool.acquire(1000), pool.acquire(600)
    assert a.numel() == 1000 and pool.stats.misses == 2 and pool.stats.bytes_in_use == 1600
    pool.release(a)
    pool.release(b)
    assert pool.stats.bytes_pooled == 1600 and pool.stats.bytes_in_use == 0
    c = pool.acquire(500)                    # both fit; the 600-byte buffer is the tighter one
    assert c.data_ptr() == b.data_ptr() and pool.stats.hits == 1
    d = pool.acquire(100)                    # 1000 bytes would waste more than 2x: a fresh buffer
    assert d.data_ptr() != a.data_ptr() and pool.stats.misses == 3
    t = pool.acquire_like((4, 8), torch.bfloat16)
    assert t.shape == (4, 8) and t.dtype == torch.bfloat16
    pool.release(t)
    assert pool.get_stats()["buffers"]["small"] == 2
    big = pool.acquire(3500)
    pool.release(big)                        # 3500 + 1000 + 64 > 4096: the oldest released buffers go
    assert pool.stats.evictions >= 1 and pool.stats.bytes_pooled <= 4096
    assert 0 < pool.stats.hit_rate < 1
    import time
    assert pool.cleanup_old_buffers(now=time.monotonic() + 60) >= 1 and pool.stats.bytes_pooled == 0
    assert BufferPool.tier_of(2 << 20) == "medium" and BufferPool.tier_of(1 << 30) == "large"


def test_transfer_stream_cpu_passthrough_and_ring_buffer():
    ts = TransferStream("cpu")
    out, ev = ts.transfer_async({"w": torch.arange(6).view(2, 3)})
    ts.wait(ev)
    ts.synchronize()
    assert ev is None and out["w"].tolist() == [[0, 1, 2], [3, 4, 5]]
    ring = RingBuffer("cpu", capacity=1024)
    x = ring.alloc((10,), torch.float32)
    y = ring.alloc((3, 4), torch.bfloat16)
    assert x.numel() == 10 and y.shape == (3, 4) and y.data_ptr() % 128 == ring.slab.data_ptr() % 128
    assert ring.used == 128 + 24 and ring.can_alloc(512) and not ring.can_alloc(1000)
    ring.reset()
    assert ring.used == 0 and ring.high_water_mark == 152 and ring.stats()["available"] == 1024
    assert get_ring_buffer("cpu", 4096) is get_ring_buffer("cpu")
    get_ring_buffer("cpu").alloc((8,), torch.uint8)
    reset_ring_buffer("cpu")
    assert get_ring_buffer("cpu").used == 0


def test_tile_coordinator_matches_the_fp4_tile_layout():
    from metal_marlin_b200.formats import fp4 as fp4fmt
    from metal_marlin_b200.memory import TileCoordinator
    tc = TileCoordinator((40, 200))
    assert (tc.num_row_tiles, tc.num_col_tiles, tc.num_tiles) == (3, 4, 12)
    assert tc.tile_to_coords(5) == (1, 1) and tc.coords_to_tile(2, 3) == 11
    rows, cols = tc.tile_bounds(11)
    assert (rows.start, rows.stop, cols.start, cols.stop) == (32, 40, 192, 200)
    assert tc.tiles_for_rows(16, 33) == [4, 5, 6, 7, 8, 9, 10, 11] and tc.tile_nbytes() == 512 and tc.byte_offset(3) == 1536
    assert [t[0] for t in tc.iter_tiles()] == list(range(12))
    # the same grid as the device layout of a quantized matrix
    codes, scales = fp4fmt.quantize_codes(torch.randn(48, 256), 64)
    qtile, _stile, _gs = fp4fmt.to_tile_layout(codes, scales)
    full = TileCoordinator((48, 256))
    assert qtile.shape[:2] == (full.num_row_tiles, full.num_col_tiles) and qtile[0, 0].numel() * 4 == full.tile_nbytes()
    import pytest
    with pytest.raises(IndexError):
        tc.tile_to_coords(12)
