"""Checkpoint maintenance (``checkpoint_tools.py`` and the ``checkpoint`` CLI group): verify / repair of MMFP4 checkpoints,
trellis container migration, base and router extraction, 2:4 pruning and draft-model creation.  Parity: reference
``scripts/{repair_mmfp4_checkpoint,migrate_trellis_v2_to_v3,extract_base_weights,extract_router_weights,prune_model,
create_draft_weights}.py``."""
import json
import os

import pytest
import torch

from metal_marlin_b200 import checkpoint_tools as ct
from metal_marlin_b200.formats.safetensors_io import load_file, save_file
from metal_marlin_b200.models.config import get_preset
from metal_marlin_b200.quant.convert import random_hf_state, save_random_checkpoint


def _float_ckpt(path, preset="tiny-mla-moe", seed=0):
    cfg = get_preset(preset)
    os.makedirs(path, exist_ok=True)
    save_file(random_hf_state(cfg, seed), os.path.join(path, "model.safetensors"), metadata={"format": "pt"})
    cfg.save_pretrained(path)
    return cfg


def test_verify_and_repair_mmfp4(tmp_path):
    d = str(tmp_path / "q")
    save_random_checkpoint(get_preset("tiny-mla-moe"), d, fmt="mmfp4", seed=1)
    rep = ct.verify_mmfp4_checkpoint(d)
    assert rep["ok"] and rep["tensors"] > 20 and not rep["unpaired"] and not rep["shape_mismatch"]
    # damage: a non-finite scale, a lost norm tensor, and an index that names a tensor no shard holds
    shard = sorted(f for f in os.listdir(d) if f.endswith(".safetensors"))[0]
    t = load_file(os.path.join(d, shard))
    sk = next(k for k in t if k.endswith(".scales"))
    t[sk] = t[sk].clone()
    t[sk].view(-1)[0] = float("inf")
    nk = next(k for k in t if "input_layernorm" in k)
    del t[nk]
    save_file(t, os.path.join(d, shard))
    with open(os.path.join(d, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {}, "weight_map": {**{k: shard for k in t}, "model.ghost.weight": shard}}, f)
    rep = ct.verify_mmfp4_checkpoint(d)
    assert not rep["ok"] and rep["bad_scales"] == [sk] and rep["missing"] == ["model.ghost.weight"]
    fl = str(tmp_path / "float")
    _float_ckpt(fl, seed=1)
    out = ct.repair_mmfp4_checkpoint(d, base_from=fl)
    assert out["after"]["ok"], out["after"]
    assert any("non-finite" in a for a in out["actions"]) and any("base tensors" in a for a in out["actions"])
    merged = {}
    for s in sorted(f for f in os.listdir(d) if f.endswith(".safetensors")):
        merged.update(load_file(os.path.join(d, s)))
    assert nk in merged and bool(torch.isfinite(merged[sk].float()).all())
    assert ct.repair_mmfp4_checkpoint(d, dry_run=True)["actions"] == ["dry run"]
    # the repaired checkpoint loads and runs
    from metal_marlin_b200.models.mmfp4_causal_lm import MMFP4ForCausalLM
    lm = MMFP4ForCausalLM.from_pretrained(d, "cpu")
    assert len(lm.generate([[1, 2, 3, 4]], max_new_tokens=3)[0]) == 3


def test_extract_base_and_router_weights(tmp_path):
    d = str(tmp_path / "q")
    save_random_checkpoint(get_preset("tiny-mla-moe"), d, fmt="mmfp4", seed=2)
    info = ct.extract_base_weights(d, str(tmp_path / "base.safetensors"))
    base = load_file(str(tmp_path / "base.safetensors"))
    assert info["tensors"] == len(base) > 0
    assert any("embed_tokens" in k for k in base) and any("norm" in k for k in base)
    assert all(v.dtype not in (torch.int32, torch.uint8) for v in base.values()) and not any(k.endswith(".scales") for k in base)
    ct.extract_base_weights(d, str(tmp_path / "router.safetensors"), routers=True)
    r = load_file(str(tmp_path / "router.safetensors"))
    assert r and all("mlp.gate" in k for k in r)


def test_trellis_container_migration_round_trip(tmp_path):
    from metal_marlin_b200.formats.trellis import TrellisModelLoader, quantize_model_trellis
    fl = str(tmp_path / "float")
    _float_ckpt(fl, preset="tiny-llama")
    v3 = str(tmp_path / "v3")
    quantize_model_trellis(fl, v3, bits=3, group_size=64, container="v3")
    v2 = str(tmp_path / "v2")
    info = ct.migrate_trellis(v3, v2, to="v2")
    assert info["from"] == "v3_hf_shards" and info["to"] == "v2_layers" and info["weights"] > 0
    back = str(tmp_path / "v3b")
    info2 = ct.migrate_trellis(v2, back, to="v3")
    assert info2["to"] == "v3_hf_shards" and info2["bits"] == info["bits"]
    a, b = TrellisModelLoader(v3), TrellisModelLoader(back)
    assert sorted(a.weight_names()) == sorted(b.weight_names())
    n = a.weight_names()[0]
    wa, wb = a.load_weight(n), b.load_weight(n)
    assert torch.equal(wa.indices, wb.indices) and torch.equal(wa.scales, wb.scales) and wa.shape == wb.shape
    assert os.path.isfile(os.path.join(back, "config.json"))
    base_key = next(k for k in a._where if "norm" in k)
    assert torch.equal(a.load_tensor(base_key), b.load_tensor(base_key))


def test_prune_checkpoint_and_create_draft(tmp_path):
    fl = str(tmp_path / "float")
    cfg = _float_ckpt(fl, preset="tiny-llama")
    pr = str(tmp_path / "pruned")
    info = ct.prune_checkpoint_24(fl, pr)
    assert info["pruned_matrices"] > 0 and abs(info["density"] - 0.5) < 1e-3
    t = load_file(os.path.join(pr, "model.safetensors"))
    w = t["model.layers.0.self_attn.q_proj.weight"].float()
    assert bool(((w.reshape(w.shape[0], -1, 4) != 0).sum(-1) <= 2).all())
    assert torch.equal(t["model.norm.weight"], load_file(os.path.join(fl, "model.safetensors"))["model.norm.weight"])
    dr = str(tmp_path / "draft")
    info = ct.create_draft_checkpoint(fl, dr, num_layers=1)
    assert info["layers"] == [0]
    dcfg = json.load(open(os.path.join(dr, "config.json")))
    assert dcfg["num_hidden_layers"] == 1 and cfg.num_hidden_layers == 2
    dt = load_file(os.path.join(dr, "model.safetensors"))
    assert any(k.startswith("model.layers.0.") for k in dt) and not any(k.startswith("model.layers.1.") for k in dt)
    assert "model.embed_tokens.weight" in dt
    # the last layer alone, renumbered
    ct.create_draft_checkpoint(fl, str(tmp_path / "d2"), layers=[1])
    d2 = load_file(os.path.join(str(tmp_path / "d2"), "model.safetensors"))
    src = load_file(os.path.join(fl, "model.safetensors"))
    assert torch.equal(d2["model.layers.0.mlp.down_proj.weight"], src["model.layers.1.mlp.down_proj.weight"])


def test_checkpoint_cli(tmp_path):
    from click.testing import CliRunner
    from metal_marlin_b200.cli import cli
    d = str(tmp_path / "q")
    save_random_checkpoint(get_preset("tiny-llama"), d, fmt="mmfp4", seed=3)
    r = CliRunner().invoke(cli, ["checkpoint", "verify", d])
    assert r.exit_code == 0 and json.loads(r.output.strip().splitlines()[-1])["ok"]
    r = CliRunner().invoke(cli, ["checkpoint", "extract", d, str(tmp_path / "b.safetensors")])
    assert r.exit_code == 0 and json.loads(r.output.strip().splitlines()[-1])["tensors"] > 0
    r = CliRunner().invoke(cli, ["checkpoint", "create-draft", d, str(tmp_path / "dr"), "--num-layers", "1"])
    assert r.exit_code == 0 and os.path.isfile(os.path.join(str(tmp_path / "dr"), "model.safetensors"))
