"""Vision front end (reference: tests/test_vision_preprocess.py, test_vision_projector.py)."""
import pytest
import torch
import torch.nn.functional as F

from metal_marlin_b200 import vision as V


def test_preprocessor_shapes_and_values():
    img = torch.randint(0, 256, (2, 50, 70, 3), dtype=torch.uint8)
    pre = V.ImagePreprocessor(V.PreprocessConfig(image_size=28, patch_size=14))
    p = pre(img)
    assert p.shape == (2, 4, 3 * 14 * 14) and pre.num_patches() == 4
    pix = V.ImagePreprocessor(V.PreprocessConfig(image_size=28, patch_size=14, as_patches=False))(img)
    assert pix.shape == (2, 3, 28, 28)
    # patch (0, 1) channel 2 equals the corresponding window of the CHW output
    torch.testing.assert_close(p[0, 1].view(3, 14, 14)[2], pix[0, 2, :14, 14:28])
    white = torch.full((1, 8, 8, 3), 255, dtype=torch.uint8)
    out = V.ImagePreprocessor(V.PreprocessConfig(image_size=8, patch_size=8, as_patches=False, mean=(0.5, 0.5, 0.5), std=(0.5, 0.5, 0.5)))(white)
    assert torch.allclose(out.float(), torch.ones(1, 3, 8, 8), atol=1e-2)
    assert V.dynamic_tiles(448, 896) == (1, 2) and V.dynamic_tiles(896, 448) == (2, 1)


def test_projectors_and_token_merge():
    torch.manual_seed(0)
    feats = torch.randn(2, 16, 32)
    llava = V.LlavaProjector(torch.randn(64, 32) * 0.1, torch.zeros(64), torch.randn(48, 64) * 0.1, torch.zeros(48))
    assert llava(feats).shape == (2, 16, 48)
    merger = V.PatchMergerProjector(torch.ones(32), torch.zeros(32), torch.randn(64, 128) * 0.1, torch.zeros(64), torch.randn(48, 64) * 0.1,
                                    torch.zeros(48), merge=2)
    assert merger(feats, (4, 4)).shape == (2, 4, 48)
    shuf = V.PixelShuffleProjector(torch.ones(128), torch.zeros(128), torch.randn(64, 128) * 0.1, torch.zeros(64), torch.randn(48, 64) * 0.1,
                                   torch.zeros(48), scale=0.5)
    assert shuf(feats).shape == (2, 4, 48)
    res = V.PerceiverResampler(torch.randn(6, 32), *(torch.randn(32, 32) * 0.1 for _ in range(4)), n_heads=4)
    assert res(feats).shape == (2, 6, 32)
    ids = torch.tensor([[1, 9, 9, 2], [9, 9, 3, 4]])
    text = torch.zeros(2, 4, 8)
    merged = V.merge_image_tokens(text, torch.ones(2, 2, 8), ids, image_token_id=9)
    assert merged[0, 1].sum() == 8 and merged[0, 0].sum() == 0 and merged[1, 2].sum() == 0


def test_encoder_cache_and_quant_config():
    cache = V.VisionEncoderCache(max_entries=2)
    calls = []
    enc = lambda im: calls.append(1) or im.float().mean().view(1)
    a, b, c = (torch.full((4, 4, 3), v, dtype=torch.uint8) for v in (1, 2, 3))
    cache.get_or_encode(a, enc), cache.get_or_encode(a, enc), cache.get_or_encode(b, enc), cache.get_or_encode(c, enc), cache.get_or_encode(a, enc)
    assert len(calls) == 4 and cache.hits == 1
    q = V.VisionQuantConfig()
    assert q.should_quantize("blocks.0.attn.qkv.weight", (768, 768)) and not q.should_quantize("patch_embed.proj.weight", (768, 588))
    assert not q.should_quantize("blocks.0.norm1.weight", (768,))


def test_general_preprocessing_cpu_semantics():
    """Crop + resample + merge-group patch order of the general preprocessing op (CPU restatement) and the dynamic
    resolution rule."""
    import torch
    from metal_marlin_b200 import ops
    from metal_marlin_b200.vision import center_crop_box, channel_statistics, preprocess_dynamic, smart_resize
    assert center_crop_box(100, 160) == (0, 30, 100, 100) and center_crop_box(160, 100) == (30, 0, 100, 100)
    assert smart_resize(100, 100) == (112, 112)
    h, w = smart_resize(1000, 500, max_pixels=28 * 28 * 100)
    assert h % 28 == 0 and w % 28 == 0 and h * w <= 28 * 28 * 100 and abs(h / w - 2.0) < 0.3
    img = torch.randint(0, 256, (2, 60, 90, 3), dtype=torch.uint8)
    out = ops.vision_preprocess_ex(img, 28, 28, crop=center_crop_box(60, 90), patch=7, merge=2, resample="bicubic")
    assert out.shape == (2, 16, 3 * 49)
    plain = ops.vision_preprocess_ex(img, 28, 28, crop=center_crop_box(60, 90), patch=7, merge=1, resample="bicubic")
    # merge order: patch (py, px) sits at ((py // 2) * 2 + px // 2) * 4 + (py % 2) * 2 + px % 2
    for py in range(4):
        for px in range(4):
            j = ((py // 2) * 2 + px // 2) * 4 + (py % 2) * 2 + px % 2
            assert torch.equal(out[:, j], plain[:, py * 4 + px])
    st = channel_statistics(img)
    v = img.float() / 255
    assert torch.allclose(st[..., 0], v.mean((1, 2)), atol=1e-5) and torch.allclose(st[..., 1], v.std((1, 2), unbiased=False), atol=1e-5)
    patches, grid = preprocess_dynamic(img[0], patch=14, merge=2)
    assert patches.shape[0] == grid[0] * grid[1] and grid[0] % 2 == 0 and grid[1] % 2 == 0


@pytest.mark.gpu
@pytest.mark.parametrize("resample", ["bilinear", "bicubic", "nearest"])
def test_general_preprocessing_kernel_matches_restatement(resample):
    import torch
    from metal_marlin_b200 import ops
    from metal_marlin_b200.vision import center_crop_box, channel_statistics
    torch.manual_seed(0)
    img = torch.randint(0, 256, (3, 75, 131, 3), dtype=torch.uint8, device="cuda")
    for (oh, ow, patch, merge, crop) in [(56, 84, 0, 1, None), (56, 56, 14, 2, center_crop_box(75, 131)), (112, 28, 7, 1, (5, 9, 60, 100))]:
        got = ops.vision_preprocess_ex(img, oh, ow, crop=crop, patch=patch, merge=merge, resample=resample).float()
        with ops.force_reference():
            want = ops.vision_preprocess_ex(img, oh, ow, crop=crop, patch=patch, merge=merge, resample=resample).float()
        assert got.shape == want.shape
        assert float((got - want).abs().max()) < 4e-2, (resample, oh, ow)
    st = channel_statistics(img)
    v = img.float() / 255
    assert torch.allclose(st[..., 0], v.mean((1, 2)), atol=1e-4) and torch.allclose(st[..., 1], v.std((1, 2), unbiased=False), atol=1e-4)
