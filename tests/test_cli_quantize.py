"""``metal-marlin`` CLI and the offline quantization driver (reference: tests/test_cli.py, test_quantize_cli.py,
test_mr_gptq_pipeline.py)."""
import json
import os

import pytest
import torch
from click.testing import CliRunner

from metal_marlin_b200.cli import cli
from metal_marlin_b200.formats.safetensors_io import save_file
from metal_marlin_b200.models.config import get_preset
from metal_marlin_b200.quant.convert import random_hf_state
from metal_marlin_b200.quant.pipeline import collect_hessians, quantize_checkpoint


@pytest.fixture()
def float_ckpt(tmp_path):
    cfg = get_preset("tiny-mla-moe")
    d = str(tmp_path / "float")
    os.makedirs(d)
    save_file(random_hf_state(cfg, seed=5), os.path.join(d, "model.safetensors"), metadata={"format": "pt"})
    cfg.save_pretrained(d)
    return cfg, d


def test_hessians_cover_dense_and_expert_tensors(float_ckpt, tmp_path):
    cfg, d = float_ckpt
    rtn_dir = str(tmp_path / "rtn")
    quantize_checkpoint(d, rtn_dir, fmt="mmfp4", method="rtn", group_size=64, device="cpu")
    col = collect_hessians(rtn_dir, "synthetic", num_samples=2, seq_len=24, device="cpu")
    names = col.names()
    assert "model.layers.0.self_attn.q_a_proj.weight" in names and "model.layers.0.self_attn.o_proj.weight" in names
    assert any(".experts." in n and n.endswith("down_proj.weight") for n in names)
    assert any("shared_experts.gate_proj" in n for n in names)
    H = col.get("model.layers.0.self_attn.o_proj.weight")
    assert H.shape[0] == H.shape[1] and torch.allclose(H, H.t(), atol=1e-4) and float(torch.diag(H).min()) >= 0


@pytest.mark.parametrize("method", ["gptq", "mr-gptq", "awq"])
def test_calibrated_quantization_writes_a_loadable_checkpoint(float_ckpt, tmp_path, method):
    cfg, d = float_ckpt
    out = str(tmp_path / method)
    st = quantize_checkpoint(d, out, fmt="mmfp4", method=method, group_size=64, num_samples=2, seq_len=24, device="cpu")
    assert st["method"] == method
    if method == "awq":        # one scale per (norm -> projections) group, folded into the weights and out of the norm
        assert st["awq_groups"] >= 2 * cfg.num_hidden_layers and st["awq_scaled_tensors"] >= 4 * cfg.num_hidden_layers
        assert st["awq_mean_gain"] >= 1.0
    else:
        assert st["with_hessian"] > 0 and st["quantized"] == st["with_hessian"] + st["rtn_fallback"]
    from metal_marlin_b200.models.mmfp4_causal_lm import MMFP4ForCausalLM
    lm = MMFP4ForCausalLM.from_pretrained(out, device="cpu")
    assert torch.isfinite(lm.forward_logits(list(range(5, 21)))).all()
    if method != "awq":
        assert os.path.exists(os.path.join(out, "quantize_state.json"))


def test_cli_end_to_end(float_ckpt, tmp_path):
    cfg, d = float_ckpt
    r = CliRunner()
    out = str(tmp_path / "q")
    res = r.invoke(cli, ["quantize", d, "-o", out, "--format", "mmfp4", "--group-size", "64", "--device", "cpu"])
    assert res.exit_code == 0, res.output
    assert json.loads(res.output.strip().splitlines()[-1])["quantized"] > 0
    res = r.invoke(cli, ["mmfp4", "inspect", out])
    assert res.exit_code == 0 and json.loads(res.output)["quantized"] > 0, res.output
    res = r.invoke(cli, ["generate", out, "-p", "hello", "-n", "4", "--device", "cpu"])
    assert res.exit_code == 0, res.output
    res = r.invoke(cli, ["quality", out, "--tokens", "64", "--max-length", "32", "--stride", "16", "--device", "cpu"])
    assert res.exit_code == 0 and json.loads(res.output.strip().splitlines()[-1])["tokens"] == 63, res.output
    res = r.invoke(cli, ["analyze", out, "--tokens", "32", "--device", "cpu"])
    assert res.exit_code == 0 and len(json.loads(res.output.strip().splitlines()[-1])["load_imbalance"]) == cfg.num_hidden_layers, res.output
    res = r.invoke(cli, ["quantize", d, "-o", str(tmp_path / "t"), "--format", "trellis-v2", "--bits", "4", "--device", "cpu"])
    assert res.exit_code == 0 and json.loads(res.output.strip().splitlines()[-1])["format"].startswith("trellis"), res.output
    res = r.invoke(cli, ["quantize", d, "-o", str(tmp_path / "i4"), "--format", "int4", "--device", "cpu"])
    assert res.exit_code == 0, res.output
    res = r.invoke(cli, ["convert", "-i", d, "-o", str(tmp_path / "c"), "--to-format", "marlin", "--quant", "fp4", "--group-size", "64"])
    assert res.exit_code == 0, res.output
    res = r.invoke(cli, ["serve"])
    assert res.exit_code != 0 and "model path" in res.output
    assert r.invoke(cli, ["--help"]).exit_code == 0


def test_serve_profiles_set_family_defaults(monkeypatch):
    import metal_marlin_b200.serving.server as srv
    seen = {}
    monkeypatch.setattr(srv, "run_server", lambda cfg, host, port, metrics_port: seen.update(cfg=cfg, port=port))
    monkeypatch.setenv("GLM47_PORT", "8123")
    r = CliRunner().invoke(cli, ["serve", "--profile", "glm47", "--batch-size", "24"])
    assert r.exit_code == 0, r.output
    cfg = seen["cfg"]
    assert (cfg.preset, cfg.num_kv_blocks, cfg.block_size, cfg.max_batch_size, cfg.max_model_len) == ("glm-4.7-flash", 4096, 16, 24, 8192)
    assert seen["port"] == 8123
    monkeypatch.setenv("GLM47_MODEL_PATH", "/models/glm")
    r = CliRunner().invoke(cli, ["serve", "--profile", "glm47", "--port", "9000", "--num-kv-blocks", "1024"])
    assert r.exit_code == 0 and seen["cfg"].model_path == "/models/glm" and seen["cfg"].preset is None
    assert seen["port"] == 9000 and seen["cfg"].num_kv_blocks == 1024 and seen["cfg"].max_batch_size == 32


def test_analysis_commands(tmp_path):
    import json
    import torch
    from metal_marlin_b200.formats.safetensors_io import save_file
    r = CliRunner()
    out = r.invoke(cli, ["analyze-routing", "--simulate", "mixtral", "--samples", "64", "--output-dir", str(tmp_path / "routing")])
    assert out.exit_code == 0, out.output
    assert "MoE routing: 32 layers x 8 experts" in out.output and (tmp_path / "routing" / "routing_report.json").is_file()
    assert r.invoke(cli, ["analyze-routing"]).exit_code != 0 and r.invoke(cli, ["analyze-routing", "--log", "x.jsonl"]).exit_code != 0
    torch.manual_seed(0)
    f = str(tmp_path / "w.safetensors")
    save_file({"a.weight": torch.randn(32, 128) * 0.05, "b.weight": torch.randn(16, 64) * 0.05, "n.weight": torch.ones(64)}, f)
    out = r.invoke(cli, ["error-report", f, "-o", str(tmp_path / "err"), "--formats", "fp4,int8", "--group-size", "64"])
    assert out.exit_code == 0, out.output
    assert "fp4: 2 matrices" in out.output and "int8: 2 matrices" in out.output
    rep = json.load(open(tmp_path / "err" / "error_report.json"))
    assert set(rep["layers"]) == {"a.weight", "b.weight"}
    out = r.invoke(cli, ["flops", "--preset", "glm-4.7-flash", "--top", "3"])
    assert out.exit_code == 0 and "lm_head" in out.output and "TFLOP" in out.output
    assert r.invoke(cli, ["flops"]).exit_code != 0
