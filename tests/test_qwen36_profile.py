"""Qwen3.6-27B shape contract (reference ``tests/test_qwen36_27b_profile.py``: dimensions, layer pattern, config parsing,
detection of the dense model, payload)."""
import dataclasses
import json

import pytest

from metal_marlin_b200.models import qwen36_profile as qp

HF = {"model_type": "qwen3_5", "_name_or_path": "Qwen/Qwen3.6-27B",
      "text_config": {"model_type": "qwen3_5_text", "hidden_size": 5120, "num_hidden_layers": 64, "vocab_size": 248320, "max_position_embeddings": 262144,
                      "full_attention_interval": 4, "rms_norm_eps": 1e-6, "linear_num_key_heads": 16, "linear_num_value_heads": 48,
                      "linear_key_head_dim": 128, "linear_value_head_dim": 128, "linear_conv_kernel_dim": 4, "num_attention_heads": 24,
                      "num_key_value_heads": 4, "head_dim": 256, "partial_rotary_factor": 0.25, "intermediate_size": 17408}}


def test_default_profile_dimensions():
    p = qp.QWEN36_27B_PROFILE
    assert p.delta.q_features == 2048 and p.delta.v_features == 6144 and p.delta.beta_features == 48 and p.delta.state_elements == 48 * 128 * 128
    assert p.attention.q_features == 24 * 256 * 2 and p.attention.kv_features == 1024 and p.attention.o_features == 6144 and p.attention.rotary_dim == 64
    assert p.full_attention_layer_indices[:3] == [3, 7, 11] and p.num_full_attention_layers == 16 and p.num_linear_attention_layers == 48
    assert p.layer_types.count("linear_attention") == 48 and p.layer_types[3] == "full_attention"
    assert 26e9 < p.weight_elements() < 29e9                                       # "27B"
    assert p.kv_bytes_per_token() == 2 * 16 * 1024 * 2 and p.recurrent_state_bytes(2) == 2 * p.recurrent_state_bytes(1)
    assert p.hardware.sms == 148 and len(p.hardware.rules) >= 5
    with pytest.raises(dataclasses.FrozenInstanceError):
        p.hidden_size = 1


def test_parse_detect_and_payload(tmp_path):
    p = qp.profile_from_hf_config(HF)
    assert p == dataclasses.replace(qp.QWEN36_27B_PROFILE, model_id="Qwen/Qwen3.6-27B") and qp.is_qwen36_27b_profile(p)
    assert qp.is_qwen36_27b_config(HF) and qp.is_qwen36_27b_config(HF["text_config"], "some/Qwen3.6-27B-int4")
    assert not qp.is_qwen36_27b_config(HF, "Qwen/Qwen3.6-35B-A3B") and not qp.is_qwen36_27b_config({"hidden_size": 5120})
    moe = json.loads(json.dumps(HF))
    moe["text_config"]["num_experts"] = 128
    assert not qp.is_qwen36_27b_config(moe)
    other = json.loads(json.dumps(HF))
    other["text_config"]["num_hidden_layers"] = 48
    po = qp.profile_from_hf_config(other)
    assert not qp.is_qwen36_27b_profile(po)
    with pytest.raises(ValueError, match="num_hidden_layers: 48"):
        qp.validate_supported_profile(po)
    qp.validate_supported_profile(p)
    # interval derived from an explicit layer list
    listed = json.loads(json.dumps(HF["text_config"]))
    del listed["full_attention_interval"]
    listed["layer_types"] = ["linear_attention", "linear_attention", "linear_attention", "full_attention"] * 16
    assert qp.profile_from_hf_config(listed).full_attention_interval == 4
    f = tmp_path / "config.json"
    f.write_text(json.dumps(HF))
    assert qp.load_profile_from_config_file(str(f)) == p
    f.write_text("[1]")
    with pytest.raises(ValueError):
        qp.load_profile_from_config_file(str(f))
    pay = qp.shape_contract_payload(p)
    assert pay["mlp_kind"] == "dense" and pay["weights_loaded"] is False and pay["num_full_attention_layers"] == 16 and pay["delta"]["value_heads"] == 48
    assert json.loads(json.dumps(pay))["hardware"]["warp_size"] == 32


def test_profile_to_engine_config_and_artifact_shapes():
    from metal_marlin_b200.converters import qmi4
    cfg = qp.QWEN36_27B_PROFILE.to_model_config()
    assert cfg.layer_types == qp.QWEN36_27B_PROFILE.layer_types and cfg.vocab_size == 248320 and cfg.layer_is_linear(0) and not cfg.layer_is_linear(3)
    shapes = qmi4.role_shapes(cfg)
    assert shapes["linear_attn_v"] == (5120, 6144) and shapes["mlp_down"] == (17408, 5120) and shapes["lm_head"] == (5120, 248320)
    assert shapes["full_attn_k"] == (5120, 1024)
