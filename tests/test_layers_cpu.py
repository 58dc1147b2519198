"""Quantized linear layers on CPU (PyTorch restatement path) — reference: tests/test_mmfp4_linear.py,
test_trellis_linear.py, test_quantized_linear*.py."""
import pytest
import torch

from metal_marlin_b200.formats import fp4 as fp4fmt
from metal_marlin_b200.layers import HadamardLinear, MMFP4Linear, QuantizedLinear, TrellisLinear
from metal_marlin_b200.quant import gptq, hadamard


def test_mmfp4_linear_from_checkpoint_tensors_both_orientations():
    torch.manual_seed(0)
    w = torch.randn(32, 128) * 0.05
    codes, scales = fp4fmt.quantize_codes(w, 64)
    ref = fp4fmt.dequantize_codes(codes, scales)
    x = torch.randn(3, 128).to(torch.bfloat16)
    for layout, pack in (("mmfp4", fp4fmt.pack_mmfp4), ("marlin_fp4", fp4fmt.pack_marlin_fp4)):
        packed, sc = pack(codes, scales)
        lin = MMFP4Linear.from_pretrained_weight(packed, sc, layout=layout)
        torch.testing.assert_close(lin(x).float(), x.float() @ ref.t(), rtol=2e-2, atol=2e-2)
        torch.testing.assert_close(lin.dequantize(torch.float32), ref)
    lin = MMFP4Linear.from_float(w, 64, bias=torch.ones(32))
    assert lin(x.view(1, 3, 128)).shape == (1, 3, 32)


@pytest.mark.parametrize("fmt", ["int8", "int4", "int3", "int2", "fp8", "nf4", "nf3", "nf2"])
def test_quantized_linear_formats(fmt):
    torch.manual_seed(1)
    w = torch.randn(24, 256) * 0.05
    lin = QuantizedLinear.from_float(w, fmt, group_size=64)
    from metal_marlin_b200.quant.rtn import quantize
    ref = quantize(w, fmt, 64).dequantize()
    torch.testing.assert_close(lin.dequantize(torch.float32), ref, rtol=1e-3, atol=1e-4)
    x = torch.randn(4, 256).to(torch.bfloat16)
    torch.testing.assert_close(lin(x).float(), x.float() @ ref.t(), rtol=3e-2, atol=3e-2)
    assert lin(torch.randn(20, 256)).shape == (20, 24)


@pytest.mark.parametrize("bits", [2, 4, 6])
def test_trellis_linear(bits):
    torch.manual_seed(2)
    w = torch.randn(48, 160) * 0.05
    lin = TrellisLinear.from_float(w, bits, group_size=32)
    deq = lin.dequantize(torch.float32)
    assert (deq - w).abs().max() < {2: 0.12, 4: 0.03, 6: 0.01}[bits]
    x = torch.randn(2, 160).to(torch.bfloat16)
    torch.testing.assert_close(lin(x).float(), x.float() @ deq.t(), rtol=3e-2, atol=3e-2)
    assert lin(torch.randn(12, 160)).shape == (12, 48)


def test_hadamard_linear_runs_a_rotated_weight():
    torch.manual_seed(3)
    w = torch.randn(16, 256) * 0.05
    w[:, 5] *= 30
    wq, scales, st = gptq.mr_gptq_quantize(w, None, gptq.MRGPTQConfig(fmt="fp4", group_size=128, force_rotation=True))
    qt = gptq.to_quantized_tensor(wq, scales, "fp4", 128)
    from metal_marlin_b200.ops.weights import FP4Weight
    lin = HadamardLinear(MMFP4Linear(FP4Weight.from_codes(qt.codes, qt.scales)), block=128)
    x = torch.randn(3, 256)
    y = lin(x.to(torch.bfloat16)).float()
    assert (y - x @ w.t()).abs().max() / (x @ w.t()).abs().max() < 0.15
