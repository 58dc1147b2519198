"""2:4 structured-sparse FP4 linear: pruning pattern, packing / de-quantization round trip against the C++ pruning oracle (CPU),
and the tensor-core GEMM that scatters the kept values inside its main loop (GPU)."""
import pytest
import torch

from metal_marlin_b200 import ops
from metal_marlin_b200.layers import Sparse24Linear


def test_prune_pack_roundtrip_and_storage():
    torch.manual_seed(0)
    w = torch.randn(48, 256) * 0.05
    lin = Sparse24Linear.from_float(w, 64)
    assert lin.codes.shape == (48, 64) and lin.meta.shape == (48, 32) and lin.scales.shape == (48, 4)
    assert lin.nbytes() == 48 * 256 * 3 // 8 + 48 * 4 * 2                     # 0.375 bytes per dense weight + scales
    d = lin.dequantize()
    g = d.view(48, 64, 4)
    assert int((g != 0).sum(-1).max()) <= 2                                    # at most two survivors per group of four
    # the survivors are the two largest magnitudes of each group, quantized to E2M1 on the group scale
    vals, pos = Sparse24Linear.prune(w)
    keep = torch.zeros(48, 64, 4, dtype=torch.bool).scatter_(2, pos, True)
    assert bool((g[~keep] == 0).all())
    from metal_marlin_b200.formats import fp4 as fp4fmt
    codes, scales = fp4fmt.quantize_codes(vals.reshape(48, 128), 32)
    want = fp4fmt.dequantize_codes(codes, scales).view(48, 64, 2)
    torch.testing.assert_close(g.gather(2, pos), want)
    err = (d - w * keep.view(48, 256)).abs().max()
    assert float(err) < 0.25 * float(w.abs().max())
    # the C++ oracle prunes to the same pattern
    from metal_marlin_b200 import ref
    pruned = ref.prune_2_4(w)
    pr = pruned[0] if isinstance(pruned, (tuple, list)) else pruned
    assert torch.equal(pr != 0, keep.view(48, 256)) or int(((pr != 0) != keep.view(48, 256)).sum()) <= 4     # ties
    x = (torch.randn(5, 256) * 0.5).to(torch.bfloat16)
    y = lin(x)
    torch.testing.assert_close(y.float(), (x.float() @ d.t()).to(torch.bfloat16).float())
    with pytest.raises(ValueError):
        Sparse24Linear.from_float(torch.randn(8, 96), 32)


@pytest.mark.gpu
@pytest.mark.parametrize("M,out_f,in_f,gs", [(1, 96, 256, 64), (40, 200, 1024, 128), (300, 136, 640, 32), (1100, 256, 512, 128)])
def test_sparse24_gemm_on_the_tensor_cores(M, out_f, in_f, gs):
    torch.manual_seed(3)
    dev = "cuda"
    w = torch.randn(out_f, in_f) * 0.05
    lin = Sparse24Linear.from_float(w, gs, device=dev)
    x = (torch.randn(M, in_f, device=dev) * 0.5).to(torch.bfloat16)
    y = lin(x)
    want = x.float().cpu() @ lin.dequantize().cpu().t()
    err = (y.float().cpu() - want).abs().max() / want.abs().max()
    assert err < 1.5e-2, float(err)
    assert ops.check_status(torch.device(dev)) == 0
