"""Quantizer kernels (``csrc/quantizer.cu``) against the PyTorch code they restate: the GPTQ block kernel and the fused
FP4 quantize + pack kernel must reproduce it bit for bit.  Parity: reference ``tests/test_gptq_metal.py`` /
``tests/test_quantize_fp4.py`` (device quantizers against their host implementations)."""
import pytest
import torch

from metal_marlin_b200 import ops
from metal_marlin_b200.formats import fp4 as fp4fmt
from metal_marlin_b200.quant.gptq import GPTQConfig, gptq_quantize

pytestmark = pytest.mark.gpu


def _hessian(in_f, tokens, seed, dev):
    g = torch.Generator(device="cpu").manual_seed(seed)
    x = torch.randn(tokens, in_f, generator=g) * (1.0 + 3.0 * torch.rand(in_f, generator=g))
    return (x.t() @ x / tokens).to(dev)


@pytest.mark.parametrize("fmt,out_f,in_f,gs,block,act_order", [
    ("fp4", 96, 512, 128, 128, False),
    ("fp4", 50, 320, 64, 128, True),        # ragged rows, a 64-column tail block, permuted columns
    ("int4", 64, 256, 128, 64, False),
    ("nf4", 33, 256, 64, 128, False),
    ("int8", 40, 256, 128, 128, False),     # 255-value grid
])
def test_gptq_block_kernel_equals_torch_loop(fmt, out_f, in_f, gs, block, act_order):
    dev = torch.device("cuda")
    torch.manual_seed(0)
    w = (torch.randn(out_f, in_f) * 0.05).to(dev)
    H = _hessian(in_f, 1024, 1, dev)
    cfg = GPTQConfig(fmt=fmt, group_size=gs, block_size=block, act_order=act_order)
    q_native, s_native, st_native = gptq_quantize(w, H, cfg)
    with ops.force_reference():
        q_torch, s_torch, st_torch = gptq_quantize(w, H, cfg)
    assert torch.equal(s_native, s_torch)
    assert torch.equal(q_native, q_torch), float((q_native - q_torch).abs().max())
    assert st_native["sq_err"] == pytest.approx(st_torch["sq_err"], rel=1e-4)
    # and the result is better than round-to-nearest under the Hessian metric
    d = (q_native - w).to(torch.float64)
    Hd = H.to(torch.float64)
    rtn, _, _ = gptq_quantize(w, torch.eye(in_f, device=dev), cfg)
    d0 = (rtn - w).to(torch.float64)
    assert float((d @ Hd * d).sum()) <= float((d0 @ Hd * d0).sum()) * 1.001


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("out_f,in_f,gs", [(64, 512, 128), (37, 192, 64), (16, 96, 32), (8, 48, 16), (5, 24, 8)])
def test_fp4_quantize_pack_equals_torch(dtype, out_f, in_f, gs):
    dev = torch.device("cuda")
    torch.manual_seed(out_f + in_f)
    w = (torch.randn(out_f, in_f) * 0.1).to(dtype)
    w[0, :gs] = 0                                   # an all-zero group takes the smallest scale
    w[1, 3] = 5.0                                   # an outlier that sets its group's scale
    w = w.to(dev)
    packed, scales = ops.fp4_quantize_pack(w, gs)
    ref_packed, ref_scales = fp4fmt.pack_mmfp4(*fp4fmt.quantize_codes(w, gs))
    assert torch.equal(scales, ref_scales)
    assert torch.equal(packed, ref_packed)
    # the layout helper takes the same route
    p2, s2, gs2 = fp4fmt.quantize_fp4(w, gs, layout="marlin_fp4")
    assert gs2 == gs and torch.equal(p2, ref_packed.t()) and torch.equal(s2, ref_scales.t())
