"""GGUF reader / block de-quantizers, GPTQ import, mixed-format pack and the convert command (reference:
tests/test_gguf_loader.py, test_gguf_to_marlin.py, test_converters.py, test_mixed_format.py)."""
import os
import struct

import numpy as np
import pytest
import torch

from metal_marlin_b200.converters import MixedFormatPack, convert_checkpoint, dequantize_gptq_int4, gguf


def _scalar_q4_k(block: bytes) -> np.ndarray:
    """Straightforward restatement of the Q4_K block rule, one element at a time."""
    d, dmin = np.frombuffer(block[:4], dtype=np.float16).astype(np.float32)
    s = block[4:16]
    qs = block[16:]

    def sm(j):
        if j < 4:
            return s[j] & 63, s[j + 4] & 63
        return (s[j + 4] & 0xF) | ((s[j - 4] >> 6) << 4), (s[j + 4] >> 4) | ((s[j] >> 6) << 4)

    y, is_, q = [], 0, 0
    for _ in range(4):
        sc1, m1 = sm(is_)
        sc2, m2 = sm(is_ + 1)
        for l in range(32):
            y.append(d * sc1 * (qs[q + l] & 0xF) - dmin * m1)
        for l in range(32):
            y.append(d * sc2 * (qs[q + l] >> 4) - dmin * m2)
        q += 32
        is_ += 2
    return np.array(y, dtype=np.float32)


def _scalar_q6_k(block: bytes) -> np.ndarray:
    ql, qh = block[:128], block[128:192]
    sc = np.frombuffer(block[192:208], dtype=np.int8)
    d = float(np.frombuffer(block[208:210], dtype=np.float16)[0])
    y = np.zeros(256, dtype=np.float32)
    for n in range(2):
        for l in range(32):
            is_ = l // 16
            a, b, h = ql[n * 64 + l], ql[n * 64 + l + 32], qh[n * 32 + l]
            q1 = ((a & 0xF) | (((h >> 0) & 3) << 4)) - 32
            q2 = ((b & 0xF) | (((h >> 2) & 3) << 4)) - 32
            q3 = ((a >> 4) | (((h >> 4) & 3) << 4)) - 32
            q4 = ((b >> 4) | (((h >> 6) & 3) << 4)) - 32
            s = sc[n * 8:]
            y[n * 128 + l] = d * s[is_ + 0] * q1
            y[n * 128 + l + 32] = d * s[is_ + 2] * q2
            y[n * 128 + l + 64] = d * s[is_ + 4] * q3
            y[n * 128 + l + 96] = d * s[is_ + 6] * q4
    return y


def test_k_quant_blocks_match_scalar_rules():
    rng = np.random.default_rng(0)
    for size, fn, scalar in ((144, gguf.dequant_q4_k, _scalar_q4_k), (210, gguf.dequant_q6_k, _scalar_q6_k)):
        raw = rng.integers(0, 256, size=3 * size, dtype=np.uint8)
        for b in range(3):                                    # keep the fp16 scales finite
            hdr = slice(b * size, b * size + 4) if size == 144 else slice(b * size + 208, b * size + 210)
            raw[hdr] = np.array([0.01, 0.02], dtype=np.float16).view(np.uint8)[: hdr.stop - hdr.start]
        got = fn(raw)
        want = np.concatenate([scalar(raw[b * size:(b + 1) * size].tobytes()) for b in range(3)])
        np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-6)


def test_legacy_blocks_and_mxfp4():
    x = np.random.default_rng(1).standard_normal(256).astype(np.float32)
    np.testing.assert_allclose(gguf.dequant_q8_0(gguf.quantize_q8_0(x)), x, atol=np.abs(x).max() / 100)
    np.testing.assert_allclose(gguf.dequant_q4_0(gguf.quantize_q4_0(x)), x, atol=np.abs(x).max() / 6)
    blk = np.zeros(20, dtype=np.uint8)
    blk[:4] = np.array([0.5, -1.0], dtype=np.float16).view(np.uint8)
    blk[4] = 0x21
    y = gguf.dequant_q4_1(blk)
    assert y[0] == 0.5 * 1 - 1.0 and y[16] == 0.5 * 2 - 1.0
    b5 = np.zeros(22, dtype=np.uint8)
    b5[:2] = np.array([2.0], dtype=np.float16).view(np.uint8)
    b5[2:6] = np.array([1 | (1 << 16)], dtype=np.uint32).view(np.uint8)          # high bits of elements 0 and 16
    b5[6] = 0x53
    y5 = gguf.dequant_q5_0(b5)
    assert y5[0] == (3 + 16 - 16) * 2.0 and y5[16] == (5 + 16 - 16) * 2.0 and y5[1] == -32.0
    mx = np.zeros(17, dtype=np.uint8)
    mx[0], mx[1] = 128, 0x7A                                                      # scale 2, codes 0xA (-1) and 0x7 (6)
    ym = gguf.dequant_mxfp4(mx)
    assert ym[0] == -2.0 and ym[16] == 12.0


def test_gguf_write_read_and_name_mapping(tmp_path):
    torch.manual_seed(0)
    tensors = {"token_embd.weight": torch.randn(50, 64), "blk.0.attn_q.weight": torch.randn(64, 64), "blk.0.attn_norm.weight": torch.ones(64),
               "blk.1.ffn_down.weight": torch.randn(64, 128)}
    types = {"blk.0.attn_q.weight": gguf.Q8_0, "blk.1.ffn_down.weight": gguf.Q4_0, "token_embd.weight": gguf.F16}
    p = str(tmp_path / "m.gguf")
    gguf.write_gguf(p, tensors, {"general.architecture": "llama", "llama.block_count": 2, "tokenizer.ggml.tokens": ["a", "b"]}, types)
    with gguf.GGUFReader(p) as r:
        assert r.metadata["general.architecture"] == "llama" and r.metadata["llama.block_count"] == 2
        assert r.metadata["tokenizer.ggml.tokens"] == ["a", "b"] and r.tensor_type("blk.0.attn_q.weight") == "Q8_0"
        for name, t in tensors.items():
            got = r.load_tensor(name)
            assert got.shape == t.shape
            tol = {gguf.Q8_0: 0.05, gguf.Q4_0: 0.6, gguf.F16: 2e-3}.get(types.get(name), 1e-6)
            assert (got - t).abs().max() <= tol
    assert gguf.gguf_name_to_hf("blk.3.ffn_gate.weight") == "model.layers.3.mlp.gate_proj.weight"
    assert gguf.gguf_name_to_hf("output_norm.weight") == "model.norm.weight"


def test_gptq_int4_import():
    torch.manual_seed(1)
    in_f, out_f, gs = 64, 16, 32
    codes = torch.randint(0, 16, (in_f, out_f))
    zeros = torch.randint(1, 16, (in_f // gs, out_f))
    scales = torch.rand(in_f // gs, out_f).half() * 0.1
    sh = torch.arange(0, 32, 4)
    qweight = (codes.view(in_f // 8, 8, out_f).long() << sh.view(1, 8, 1)).sum(1).to(torch.int32)
    qzeros = ((zeros - 1).view(in_f // gs, out_f // 8, 8).long() << sh.view(1, 1, 8)).sum(2).to(torch.int32)
    w = dequantize_gptq_int4(qweight, qzeros, scales)
    g = torch.arange(in_f) // gs
    want = ((codes - zeros[g]).float() * scales.float()[g]).t()
    torch.testing.assert_close(w, want)


def test_mixed_format_pack(tmp_path):
    torch.manual_seed(2)
    pack = MixedFormatPack()
    a, b, c = torch.randn(16, 128) * 0.1, torch.randn(8, 128) * 0.1, torch.randn(128)
    pack.add("a", a, "fp4", 64), pack.add("b", b, "int8", 128), pack.add("c", c, "keep")
    pack.save(str(tmp_path / "mix.safetensors"))
    back = MixedFormatPack.load(str(tmp_path / "mix.safetensors"))
    assert back.manifest["a"]["format"] == "fp4" and back.manifest["b"]["bits"] == 8
    assert (back.dequantize("a") - a).abs().max() < 0.06 and (back.dequantize("b") - b).abs().max() < 5e-3
    torch.testing.assert_close(back.dequantize("c"), c)


def test_convert_gguf_to_marlin_and_back_to_gguf(tmp_path):
    from metal_marlin_b200.models.config import get_preset
    from metal_marlin_b200.quant.convert import random_hf_state
    cfg = get_preset("tiny-llama")
    sd = random_hf_state(cfg, seed=4)
    src = tmp_path / "src"
    src.mkdir()
    inv = {v: k for k, v in gguf._GGUF_TO_HF.items()}
    gg = {}
    for k, v in sd.items():                                    # HF names -> llama.cpp names for the fixture
        parts = k.split(".")
        if parts[:2] == ["model", "layers"]:
            core = ".".join(parts[3:-1])
            gg[f"blk.{parts[2]}.{inv.get(core, core)}.{parts[-1]}"] = v
        else:
            core = ".".join(parts[:-1])
            gg[f"{inv.get(core, core)}.{parts[-1]}"] = v
    gguf.write_gguf(str(src / "model.gguf"), gg, {"general.architecture": "llama"})
    cfg.save_pretrained(str(src))
    out = tmp_path / "out"
    st = convert_checkpoint(str(src), str(out), to_format="marlin", quant="mmfp4", group_size=64)
    assert st["source_format"] == "gguf" and st["quantized"] > 0
    from metal_marlin_b200.models.mmfp4_causal_lm import MMFP4ForCausalLM
    lm = MMFP4ForCausalLM.from_pretrained(str(out), device="cpu")
    assert torch.isfinite(lm.forward_logits(list(range(8)))).all()
    st2 = convert_checkpoint(str(src), str(tmp_path / "gg2"), to_format="gguf", quant="int8")
    assert st2["format"] == "gguf" and os.path.exists(tmp_path / "gg2" / "model.gguf")
