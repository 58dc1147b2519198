"""``.qmi4`` container, artifact manifest and loading as INT4 layers (``converters/qmi4.py``).  Parity: reference
``tests/test_qwen36_27b_qmi4.py`` / ``test_qwen36_27b_artifact.py`` (container round trip, header checks, role mapping,
manifest validation and coverage)."""
import dataclasses
import os

import pytest
import torch

from metal_marlin_b200.converters import qmi4
from metal_marlin_b200.models.config import get_preset

CFG = dataclasses.replace(get_preset("tiny-hybrid-deltanet"), vocab_size=256)
SHAPES = qmi4.role_shapes(CFG)


def _tensor(role, seed=0, gs=32):
    in_f, out_f = SHAPES[role]
    torch.manual_seed(seed)
    return qmi4.quantize_to_qmi4(torch.randn(out_f, in_f) * 0.05, gs, source_key=f"model.{role}.weight")


def test_container_round_trip_and_dequantization(tmp_path):
    t = _tensor("mlp_gate")
    w = torch.manual_seed(0) and None
    p = str(tmp_path / "mlp_gate.qmi4")
    qmi4.write_qmi4_tensor(p, t)
    r = qmi4.read_qmi4_tensor(p)
    assert r.source_key == "model.mlp_gate.weight" and (r.in_features, r.out_features, r.group_size) == (*SHAPES["mlp_gate"], 32)
    assert torch.equal(r.qweight, t.qweight) and torch.equal(r.scales, t.scales) and torch.equal(r.zeros, t.zeros)
    torch.manual_seed(0)
    ref = torch.randn(SHAPES["mlp_gate"][1], SHAPES["mlp_gate"][0]) * 0.05
    deq = r.dequantize()
    assert deq.shape == ref.shape and float((deq - ref).abs().max()) < float(r.scales.float().max()) * 0.51 + 1e-6
    assert int(r.codes().max()) <= 15 and r.codes().shape == ref.shape
    # the INT4 layer computes with the same weights
    lin = r.to_linear("cpu")
    x = torch.randn(5, r.in_features)
    y = lin(x.bfloat16()).float()
    assert float((y - x.bfloat16().float() @ deq.t()).abs().max()) < 0.05 * float((x @ deq.t()).abs().max()) + 1e-3
    # damaged files are refused
    raw = bytearray(open(p, "rb").read())
    open(p, "wb").write(bytes(raw[:-2]))
    with pytest.raises(ValueError):
        qmi4.read_qmi4_tensor(p)
    raw[0:4] = b"NOPE"
    open(p, "wb").write(bytes(raw))
    with pytest.raises(ValueError):
        qmi4.read_qmi4_tensor(p)


def test_role_shapes_follow_the_configuration():
    full = qmi4.role_shapes()
    assert full["linear_attn_q"] == (5120, 16 * 128) and full["linear_attn_v"] == (5120, 48 * 128) and full["linear_attn_beta"] == (5120, 48)
    assert full["full_attn_q"] == (5120, 24 * 256) and full["full_attn_k"] == (5120, 4 * 256) and full["mlp_down"] == (17408, 5120)
    assert qmi4.expected_tensor_shape("lm_head") == (5120, 151936)
    assert qmi4.role_from_legacy_name("b.qmi4") == "linear_attn_beta" and qmi4.role_from_legacy_name("x/attn_o.qmi4") == "full_attn_o"
    with pytest.raises(ValueError):
        qmi4.role_from_legacy_name("unknown.qmi4")


def test_directory_import_manifest_and_coverage(tmp_path):
    src, out = str(tmp_path / "proto"), str(tmp_path / "artifact")
    os.makedirs(src)
    legacy = {v: k for k, v in qmi4.LEGACY_NAMES.items() if k != "beta"}
    for role in qmi4.REQUIRED_ROLES:
        qmi4.write_qmi4_tensor(os.path.join(src, legacy[role] + ".qmi4"), _tensor(role, seed=len(role)))
    m = qmi4.import_qmi4_directory(src, out, layer_index=None, shapes=SHAPES)
    assert len(m.tensors) == len(qmi4.REQUIRED_ROLES) and os.path.isfile(os.path.join(out, "manifest.json"))
    qmi4.validate_required_roles(qmi4.read_manifest(os.path.join(out, "manifest.json"), SHAPES), shapes=SHAPES)
    lin = qmi4.load_layer_linears(out, None, "cpu", SHAPES)
    assert set(lin) == set(qmi4.REQUIRED_ROLES) and lin["mlp_down"].in_features == SHAPES["mlp_down"][0]
    t = qmi4.load_artifact(out, m.index()[(None, "linear_attn_z")])
    assert torch.equal(t.qweight, _tensor("linear_attn_z", seed=len("linear_attn_z")).qweight)
    # a template manifest is not full-layer coverage; a complete per-layer manifest is
    with pytest.raises(ValueError):
        qmi4.validate_full_layer_coverage(m, CFG, SHAPES)
    arts = []
    for li in range(CFG.num_hidden_layers):
        for role in qmi4.layer_roles(CFG, li):
            i, o = SHAPES[role]
            arts.append(qmi4.Int4TensorArtifact(role, li, "q", "s", "z", i, o, 32))
    i, o = SHAPES["lm_head"]
    arts.append(qmi4.Int4TensorArtifact("lm_head", None, "q", "s", "z", i, o, 32))
    full = qmi4.ArtifactManifest(arts)
    qmi4.validate_full_layer_coverage(full, CFG, SHAPES)
    with pytest.raises(ValueError):
        qmi4.validate_full_layer_coverage(qmi4.ArtifactManifest(arts[:-3] + arts[-1:]), CFG, SHAPES)
    with pytest.raises(ValueError):          # wrong shape for the role
        qmi4.ArtifactManifest([qmi4.Int4TensorArtifact("mlp_up", 0, "q", "s", "z", 8, 8, 32)]).validate(SHAPES)
    with pytest.raises(ValueError):          # the same (layer, role) twice
        qmi4.ArtifactManifest([arts[0], arts[0]]).validate(SHAPES)


def test_artifact_parity_validation(tmp_path):
    """Kernel-path output of the INT4 layers against the float64 oracle over the packed words (reference
    ``tests/test_qwen36_27b_validation.py``: projection, MLP, full-attention, linear-block and LM-head parity)."""
    from metal_marlin_b200.converters import qmi4_validation as val
    assert val.sample_columns(5, 8) == (0, 1, 2, 3, 4)
    cols = val.sample_columns(1000, 16)
    assert len(cols) <= 16 and cols[0] == 0 and cols[-1] == 999 and 500 in cols and list(cols) == sorted(set(cols))
    with pytest.raises(ValueError):
        val.sample_columns(10, 0)
    t = _tensor("mlp_up", seed=3)
    x = torch.randn(t.in_features, generator=torch.Generator().manual_seed(1))
    want = (t.dequantize().double() @ x.double())
    assert torch.allclose(val.oracle_columns(x, t, (0, 7, t.out_features - 1)), want[[0, 7, t.out_features - 1]], atol=1e-9)

    src = str(tmp_path / "proto")
    os.makedirs(src)
    legacy = {v: k for k, v in qmi4.LEGACY_NAMES.items() if k != "beta"}
    for role in qmi4.REQUIRED_ROLES:
        qmi4.write_qmi4_tensor(os.path.join(src, legacy[role] + ".qmi4"), _tensor(role, seed=len(role)))
    out = str(tmp_path / "artifact")
    qmi4.import_qmi4_directory(src, out, layer_index=None, shapes=SHAPES)
    mlp = val.validate_mlp(out, None, max_columns=16, device="cpu", shapes=SHAPES)
    assert [r.role for r in mlp.results] == ["mlp_gate", "mlp_up", "mlp_down"] and mlp.norms["intermediate"] > 0
    mlp.assert_within(atol=8e-3, rtol=2e-2)
    att = val.validate_full_attention(out, None, max_columns=16, device="cpu", shapes=SHAPES, kv_heads=CFG.num_key_value_heads)
    assert set(att.by_role()) == set(qmi4.FULL_ATTENTION_ROLES)
    att.assert_within(atol=8e-3, rtol=2e-2)
    lin = val.validate_linear_block(out, None, max_columns=16, device="cpu", shapes=SHAPES)
    assert set(lin.by_role()) == set(qmi4.LINEAR_ATTENTION_ROLES)
    lin.assert_within(atol=8e-3, rtol=2e-2)
    head = val.validate_lm_head(out, max_columns=32, device="cpu", shapes=SHAPES)
    head.assert_within(atol=8e-3, rtol=2e-2)
    proj = val.validate_projections(out, None, roles=("linear_attn_q", "full_attn_k"), device="cpu", shapes=SHAPES)
    assert len(proj.results) == 2 and proj.max_abs_error < 8e-3 and proj.max_rel_error >= 0
    everything = val.validate_all(out, linear_layer=None, attention_layer=None, device="cpu", shapes=SHAPES)
    assert set(everything) == {"linear_block", "full_attention", "lm_head"}          # the MLP scan covers numbered layers only
    # a corrupted artifact is caught: flip the scales of one tensor on disk
    m = qmi4.read_manifest(os.path.join(out, "manifest.json"), SHAPES)
    art = m.index()[(None, "mlp_down")]
    good = val._Layer(out, None, "cpu", SHAPES)
    bad_t = good.tensors["mlp_down"]
    xin = torch.randn(bad_t.in_features, generator=torch.Generator().manual_seed(2))
    y = good.run("mlp_down", xin)
    broken = dataclasses.replace(bad_t, scales=bad_t.scales * 1.5)
    res = val.compare("mlp_down", xin, broken, y, 16)
    bv = val.BlockValidation(out, "mlp", [res])
    with pytest.raises(AssertionError):
        bv.assert_within(atol=8e-3, rtol=2e-2)
    with pytest.raises(KeyError):
        val.validate_mlp(out, 5, device="cpu", shapes=SHAPES)
    assert art.role == "mlp_down"
