"""Vision package surface: image operations object, ViT preprocessing, calibration sets, activation / Hessian collection,
sensitivity report, precision maps and the mixed-format pack of a vision-language model."""
import os

import numpy as np
import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

import metal_marlin_b200.vision as vis

REFERENCE_VISION = [
    "VisionProjector", "VisionProjectorConfig", "LLaVAProjector", "Qwen2VLProjector", "InternVLProjector", "detect_projector_type",
    "VisionCalibrationConfig", "build_vision_calibration_dataset", "collect_vision_calibration_stats", "analyze_vision_encoder_sensitivity",
    "build_vision_precision_map", "build_vlm_precision_map", "pack_vlm_mixed_format", "VisionMetal", "preprocess_for_vit",
]


def test_every_reference_name_resolves():
    for n in REFERENCE_VISION:
        assert getattr(vis, n) is not None, n
    assert set(REFERENCE_VISION) <= set(vis.__all__)
    assert vis.LLaVAProjector is vis.LlavaProjector and vis.detect_projector_type({"model_type": "qwen2_vl"}) == "qwen2_vl"


def test_image_operations():
    vd = vis.VisionMetal("cpu")
    g = torch.Generator().manual_seed(0)
    x = torch.rand(2, 3, 20, 30, generator=g)
    assert torch.allclose(vd.resize_bilinear(x, (10, 12)), F.interpolate(x, size=(10, 12), mode="bilinear", align_corners=False))
    assert torch.allclose(vd.resize_bicubic(x.numpy(), (25, 17)), F.interpolate(x, size=(25, 17), mode="bicubic", align_corners=False))
    nh = x.permute(0, 2, 3, 1).contiguous()
    assert torch.allclose(vd.resize_bilinear(nh, (10, 12), nhwc=True), vd.resize_bilinear(x, (10, 12)).permute(0, 2, 3, 1))
    mean, std = (0.5, 0.4, 0.3), (0.2, 0.25, 0.3)
    n = vd.normalize(x, mean, std)
    assert torch.allclose(n[:, 1], (x[:, 1] - 0.4) / 0.25) and torch.allclose(vd.normalize(nh, mean, std, nhwc=True), n.permute(0, 2, 3, 1))
    assert torch.allclose(vd.resize_and_normalize(x, (8, 8), mean, std), vd.normalize(vd.resize_bilinear(x, (8, 8)), mean, std), atol=1e-6)
    # uint8 images take the fused preprocessing path (bf16 out)
    u8 = torch.randint(0, 256, (2, 16, 24, 3), dtype=torch.uint8, generator=g)
    r = vd.resize_and_normalize(u8, (8, 12), mean, std, nhwc=True)
    ref = vd.resize_and_normalize(u8.permute(0, 3, 1, 2).float() / 255, (8, 12), mean, std).permute(0, 2, 3, 1)
    assert r.dtype == torch.bfloat16 and r.shape == (2, 8, 12, 3) and (r.float() - ref).abs().max() < 0.05
    assert torch.equal(vd.uint8_to_float(u8), u8.float() / 255)
    c = vd.center_crop(x, (10, 10))
    assert torch.equal(c, x[:, :, 5:15, 10:20]) and torch.equal(vd.center_crop(nh, (10, 10), nhwc=True), c.permute(0, 2, 3, 1))
    with pytest.raises(ValueError):
        vd.center_crop(x, (40, 10))
    p = vd.extract_patches(nh[:, :20, :30], 10)
    assert p.shape == (2, 6, 300) and torch.equal(p[0, 4].reshape(10, 10, 3), nh[0, 10:20, 10:20])
    with pytest.raises(ValueError):
        vd.extract_patches(nh, 7)
    h, w = vd.qwen2vl_size(1000, 3000, max_pixels=512 * 512, patch_size=14)
    assert h % 14 == 0 and w % 14 == 0 and h * w <= 512 * 512 and abs(w / h - 3) < 0.3
    assert vd.preprocess_qwen2vl(torch.rand(1, 3, 30, 60), max_pixels=14 * 14 * 2, patch_size=14).shape == (1, 3, 14, 28)
    pad = vd.resize_aspect_ratio_preserve(x, (30, 30), pad_value=-1.0)
    assert pad.shape == (2, 3, 30, 30) and (pad[:, :, :5] == -1).all() and (pad[:, :, 25:] == -1).all() and (pad[:, :, 5:25] > -1).all()


def test_preprocess_for_vit():
    g = torch.Generator().manual_seed(1)
    a = torch.randint(0, 256, (40, 50, 3), dtype=torch.uint8, generator=g)
    b = torch.randint(0, 256, (60, 30, 3), dtype=torch.uint8, generator=g)
    out = vis.preprocess_for_vit([a, b.numpy()], (32, 32), device="cpu")
    assert out.shape == (2, 3, 32, 32)
    ref = F.interpolate(a.permute(2, 0, 1)[None].float() / 255, size=(32, 32), mode="bilinear", align_corners=False)
    ref = (ref - torch.tensor((0.485, 0.456, 0.406)).view(1, 3, 1, 1)) / torch.tensor((0.229, 0.224, 0.225)).view(1, 3, 1, 1)
    assert (out[0].float() - ref[0]).abs().max() < 0.06
    f = torch.rand(3, 3, 48, 48, generator=g)
    assert vis.preprocess_for_vit(f, (24, 24), device="cpu").shape == (3, 3, 24, 24)


class _Tower(nn.Module):
    def __init__(self):
        super().__init__()
        self.vision_tower = nn.ModuleDict({"patch_embed": nn.Linear(48, 64), "qkv": nn.Linear(64, 192), "fc1": nn.Linear(64, 128), "fc2": nn.Linear(128, 64)})
        self.language = nn.Linear(64, 64)

    def forward(self, img):
        p = vis.VisionMetal("cpu").extract_patches(img.permute(0, 2, 3, 1), 4)          # [N, n, 48]
        h = self.vision_tower["patch_embed"](p)
        h = h + self.vision_tower["qkv"](h)[..., :64]
        h = h + self.vision_tower["fc2"](F.gelu(self.vision_tower["fc1"](h)))
        return self.language(h)


def test_calibration_sets_and_stats(tmp_path, monkeypatch):
    ds = vis.build_vision_calibration_dataset("synthetic", num_images=6, image_size=(16, 16), seed=3)
    assert ds.num_images == 6 and ds.get_all().shape == (6, 3, 16, 16) and 0 <= float(ds.get_all().min()) and float(ds.get_all().max()) <= 1
    assert torch.equal(ds.get_all(), vis.VisionCalibrationDataset.synthetic(6, (16, 16), 3).get_all()) and ds.memory_mb > 0
    assert [b.shape[0] for b in ds.get_batches(4)] == [4, 2] and len(list(ds.get_batches(2, max_batches=2))) == 2
    with pytest.raises(FileNotFoundError):
        monkeypatch.delenv("MMB200_COCO_DIR", raising=False)
        vis.build_vision_calibration_dataset("coco")
    with pytest.raises(ValueError):
        vis.build_vision_calibration_dataset("no-such-set")
    from PIL import Image
    d = tmp_path / "imgs" / "sub"
    d.mkdir(parents=True)
    rs = np.random.RandomState(0)
    for i in range(5):
        Image.fromarray(rs.randint(0, 256, (20 + i, 30, 3), dtype=np.uint8)).save(d / f"im{i}.png")
    monkeypatch.setenv("MMB200_COCO_DIR", str(tmp_path / "imgs"))
    coco = vis.build_vision_calibration_dataset("coco_subset", num_images=3, image_size=(16, 16))
    assert coco.num_images == 3 and coco.name == "coco" and coco.get_all().shape == (3, 3, 16, 16)
    assert vis.build_vision_calibration_dataset(str(tmp_path / "imgs"), num_images=10, image_size=(8, 8)).num_images == 5

    torch.manual_seed(0)
    model = _Tower()

    class Cfg:
        layer_prefix = "vision_tower"
    acts, hess = vis.collect_vision_calibration_stats(model, ds, Cfg(), batch_size=4, max_rows=40)
    assert set(acts) == set(hess) == {f"vision_tower.{k}.weight" for k in ("patch_embed", "qkv", "fc1", "fc2")}
    assert acts["vision_tower.qkv.weight"].shape == (40, 64) and hess["vision_tower.fc2.weight"].shape == (128, 128)
    H = hess["vision_tower.qkv.weight"]
    assert np.allclose(H, H.T, atol=1e-5) and np.linalg.eigvalsh(H.astype(np.float64)).min() > 0
    a2, h2 = vis.collect_vision_calibration_stats(model, ds, None, collect_hessians=False, forward_fn=lambda m, b: m(b))
    assert h2 == {} and "language.weight" in a2

    weights = {k: v.detach() for k, v in model.state_dict().items()}
    rep = vis.analyze_vision_encoder_sensitivity(weights, acts, hess, fp4_threshold=0.5, fp8_threshold=0.05, group_size=64)
    byname = {l.name: l for l in rep.layers}
    assert rep.num_layers == 5 and byname["vision_tower.patch_embed.weight"].recommended_precision == "bf16"
    q = byname["vision_tower.qkv.weight"]
    assert q.layer_type == vis.VisionLayerType.ATTENTION_QKV and 0 < q.fp8_error < q.fp4_error and q.recommended_precision == "fp4"
    strict = vis.analyze_vision_encoder_sensitivity(weights, acts, hess, fp4_threshold=1e-4, fp8_threshold=0.05, group_size=64)
    assert {l.name: l for l in strict.layers}["vision_tower.fc1.weight"].recommended_precision == "fp8"
    none = vis.analyze_vision_encoder_sensitivity(weights, fp4_threshold=1e-6, fp8_threshold=1e-6)
    assert set(none.get_precision_summary()) == {"bf16"} and len(none.get_by_type(vis.VisionLayerType.MLP_UP)) == 1
    assert strict.estimated_bytes() > rep.estimated_bytes() and rep.to_dict()["summary"] == rep.get_precision_summary()

    from metal_marlin_b200.compat_api import Precision
    vmap = vis.build_vision_precision_map({k: v for k, v in weights.items() if k.startswith("vision_tower")}, None, strict)
    assert vmap["vision_tower.fc1.weight"] == (Precision.FP8, 64) and vmap["vision_tower.patch_embed.weight"] == (Precision.BF16, 0)
    assert "vision_tower.fc1.bias" not in vmap
    dflt = vis.build_vision_precision_map(weights, vis.VisionQuantConfig(fmt="int8", group_size=64))
    assert dflt["vision_tower.qkv.weight"] == (Precision.INT8, 64) and dflt["vision_tower.patch_embed.weight"][0] == Precision.BF16
    full = dict(weights)
    full["model.embed_tokens.weight"] = torch.randn(32, 64)
    full["model.layers.0.mlp.up_proj.weight"] = torch.randn(128, 64)
    pm = vis.build_vlm_precision_map(full, Cfg(), vmap, llm_precision=Precision.FP4, llm_group_size=64)
    assert pm["model.layers.0.mlp.up_proj.weight"] == (Precision.FP4, 64) and pm["model.embed_tokens.weight"] == (Precision.BF16, 0)
    assert pm["vision_tower.fc1.weight"] == (Precision.FP8, 64) and pm["language.weight"] == (Precision.FP4, 64)
    out = str(tmp_path / "vlm.safetensors")
    pack = vis.pack_vlm_mixed_format(full, pm, out)
    assert os.path.isfile(out) and pack.manifest["vision_tower.fc1.weight"]["format"].startswith("fp8") and pack.manifest["model.embed_tokens.weight"]["format"] == "float"
    from metal_marlin_b200.converters import MixedFormatPack
    back = MixedFormatPack.load(out)
    w = full["model.layers.0.mlp.up_proj.weight"]
    assert float((back.dequantize("model.layers.0.mlp.up_proj.weight") - w).norm() / w.norm()) < 0.2
    assert float((back.dequantize("vision_tower.fc1.weight") - weights["vision_tower.fc1.weight"]).norm() / weights["vision_tower.fc1.weight"].norm()) < 0.05
