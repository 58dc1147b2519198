"""FP4 layouts: checkpoint pack/unpack, device tile layout, quantizer properties.
Modelled on the reference's tests/test_packed_format.py and tests/test_dequant*.py."""
import pytest
import torch

from metal_marlin_b200._compat import E2M1_VALUES
from metal_marlin_b200.formats import fp4
from metal_marlin_b200.ops import FP4ExpertBank, FP4Weight
from metal_marlin_b200.quant import rtn


def test_all_codes_roundtrip_exact():
    # every E2M1 value times a power-of-two scale must quantize to itself
    vals = torch.tensor(E2M1_VALUES).repeat(8).view(1, 128) * 0.25
    codes, scales = fp4.quantize_codes(vals, 128)
    assert torch.allclose(fp4.dequantize_codes(codes, scales), vals)


@pytest.mark.parametrize("out_f,in_f,gs", [(64, 256, 128), (48, 192, 64), (16, 64, 32), (80, 512, 128)])
def test_checkpoint_layout_roundtrip(out_f, in_f, gs):
    w = torch.randn(out_f, in_f) * 0.02
    codes, sc = fp4.quantize_codes(w, gs)
    p, s = fp4.pack_mmfp4(codes, sc)
    assert p.shape == (out_f, in_f // 8) and s.shape == (out_f, in_f // gs)
    c2, s2 = fp4.unpack_mmfp4(p, s)
    assert torch.equal(c2, codes) and torch.equal(s2, sc)
    # transposed scales are accepted too
    c3, s3 = fp4.unpack_mmfp4(p, s.t().contiguous())
    assert torch.equal(s3, sc)
    p, s = fp4.pack_marlin_fp4(codes, sc)
    assert p.shape == (in_f // 8, out_f) and s.shape == (in_f // gs, out_f)
    c4, s4 = fp4.unpack_marlin_fp4(p, s)
    assert torch.equal(c4, codes) and torch.equal(s4, sc)


def test_nibble_order_matches_reference_convention():
    # nibble i of word j is element 8j + i (LSB first)
    codes = torch.arange(16, dtype=torch.uint8).view(1, 16) % 16
    p, _ = fp4.pack_mmfp4(codes, torch.ones(1, 1, dtype=torch.float16))
    w0 = int(p[0, 0]) & 0xFFFFFFFF
    assert [(w0 >> (4 * i)) & 0xF for i in range(8)] == list(range(8))


@pytest.mark.parametrize("out_f,in_f,gs", [(64, 256, 128), (40, 192, 64), (16, 64, 16), (33, 128, 32)])
def test_tile_layout_roundtrip(out_f, in_f, gs):
    w = torch.randn(out_f, in_f)
    codes, sc = fp4.quantize_codes(w, gs)
    q, s, g = fp4.to_tile_layout(codes, sc)
    assert g == gs and q.shape[2:] == (32, 4)
    c2, s2 = fp4.from_tile_layout(q, s, out_f, in_f, gs)
    assert torch.equal(c2, codes) and torch.equal(s2, sc)


def test_tile_word_is_mma_fragment():
    # lane (g, t), word ks: the shift/mask sequence of the kernels must yield rows g / g+8, k 2t, 2t+1 (+8)
    out_f, in_f = 16, 64
    codes = torch.randint(0, 16, (out_f, in_f), dtype=torch.uint8)
    q, _, _ = fp4.to_tile_layout(codes, torch.ones(out_f, 1, dtype=torch.float16).repeat(1, 1).expand(out_f, in_f // 64).contiguous())
    for lane in (0, 5, 17, 31):
        g, t = lane // 4, lane % 4
        for ks in range(4):
            w = int(q[0, 0, lane, ks]) & 0xFFFFFFFF
            frags = []
            for j in range(4):       # register j = ((w << j) & 0x80008000) | ((w << 3j) & 0x0E000E00): sign bit 15, magnitude 11..9
                r = (((w << j) & 0x80008000) | ((w << (3 * j)) & 0x0E000E00)) & 0xFFFFFFFF
                code = lambda half: (((half >> 15) & 1) << 3) | ((half >> 9) & 7)
                frags.append((code(r & 0xFFFF), code(r >> 16)))
            k0 = ks * 16 + 2 * t
            exp = [(codes[g, k0], codes[g, k0 + 1]), (codes[g + 8, k0], codes[g + 8, k0 + 1]),
                   (codes[g, k0 + 8], codes[g, k0 + 9]), (codes[g + 8, k0 + 8], codes[g + 8, k0 + 9])]
            assert frags == [(int(a), int(b)) for a, b in exp]


def test_quantizer_error_bound_and_scale_rule():
    w = torch.randn(32, 256) * 0.02
    codes, sc = fp4.quantize_codes(w, 128)
    absmax = w.view(32, 2, 128).abs().amax(-1)
    assert torch.allclose(sc.float(), (absmax / 6).half().float())
    wd = fp4.dequantize_codes(codes, sc)
    # worst-case RTN error of E2M1 is half the largest step (1.0 in code units)
    assert ((wd - w).abs() <= sc.float().repeat_interleave(128, 1) * 1.0 + 1e-6).all()


def test_zero_weight_group():
    w = torch.zeros(16, 128)
    codes, sc = fp4.quantize_codes(w, 128)
    assert torch.all(fp4.dequantize_codes(codes, sc) == 0)


def test_group_size_fallback():
    assert fp4.pick_group_size(192, 128) == 64
    assert fp4.pick_group_size(256, 128) == 128
    with pytest.raises(ValueError):
        fp4.pick_group_size(100, 128)


def test_weight_containers():
    w = torch.randn(32, 128) * 0.05
    W = FP4Weight.from_float(w, 64)
    assert W.dequantize().shape == (32, 128)
    cat = FP4Weight.concat_rows([W, W])
    assert torch.equal(cat.dequantize()[32:], W.dequantize())
    bank = FP4ExpertBank.from_float(torch.randn(3, 32, 128), 64)
    assert bank.dequantize().shape == (3, 32, 128)
    assert torch.equal(bank.expert(1).dequantize(), bank.dequantize()[1])


@pytest.mark.parametrize("fmt", ["fp4", "int4", "nf4", "int8", "fp8", "int3", "int2", "nf3", "nf2"])
def test_rtn_quantizers(fmt):
    w = torch.randn(16, 256) * 0.02
    q = rtn.quantize(w, fmt, 64)
    rel, _ = rtn.quantization_error(w, q)
    bound = {"fp4": 0.2, "int4": 0.15, "nf4": 0.15, "int8": 0.01, "fp8": 0.05, "int3": 0.3, "int2": 0.6,
             "nf3": 0.3, "nf2": 0.6}[fmt]
    assert rel < bound, (fmt, rel)


@pytest.mark.parametrize("bits", [2, 3, 4, 5, 6, 8])
def test_bitstream_roundtrip(bits):
    codes = torch.randint(0, 2 ** bits, (7, 256), dtype=torch.uint8)
    p = rtn.pack_bits(codes, bits)
    assert p.shape == (7, 256 * bits // 8)
    assert torch.equal(rtn.unpack_bits(p, bits, 256), codes)
