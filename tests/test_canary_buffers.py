"""Canary-padded buffers: out-of-bounds stores are caught where they happen (CPU logic), and this library's kernels keep
inside their outputs on ragged shapes (GPU)."""
import pytest
import torch

from metal_marlin_b200.utils.canary import CanaryArena, CanaryViolation, guard_outputs


def test_arena_detects_writes_on_either_side():
    ar = CanaryArena("cpu", margin=64)
    t = ar.empty((5, 7), torch.float32, "t")
    assert t.shape == (5, 7) and t.is_contiguous() and t.data_ptr() % 256 == ar._blocks[0][0].data_ptr() % 256
    t.fill_(1.0)
    ar.check()
    raw, off, n, _ = ar._blocks[0]
    raw[off + n] = 0                                   # one byte past the end
    with pytest.raises(CanaryViolation, match="after the buffer"):
        ar.check()
    raw[off + n] = 0xA5
    raw[off - 3] = 1
    with pytest.raises(CanaryViolation, match="before the buffer"):
        ar.check()
    raw[off - 3] = 0xA5
    with CanaryArena("cpu") as ok:
        ok.zeros(9, torch.int32).add_(1)
    with pytest.raises(CanaryViolation):
        with CanaryArena("cpu") as bad:
            z = bad.zeros(4, torch.uint8)
            bad._blocks[0][0][bad._blocks[0][1] + 4] = 7


def test_guard_outputs_wraps_allocations_and_restores_torch():
    before = torch.empty
    with guard_outputs("cpu") as arena:
        a = torch.empty(3, 4, dtype=torch.float32, device="cpu")
        b = torch.zeros((2, 2), dtype=torch.bfloat16, device="cpu")
        c = torch.empty_like(a)
        d = torch.empty(3)                              # no device given: not guarded
        a.fill_(2.0)
        c.copy_(a)
        assert len(arena._blocks) == 3 and float(b.sum()) == 0 and d.shape == (3,)
    assert torch.empty is before
    from metal_marlin_b200 import ops
    from metal_marlin_b200.ops import FP4Weight
    w = FP4Weight.from_float(torch.randn(48, 64) * 0.05, 64)
    x = (torch.randn(5, 64) * 0.5).to(torch.bfloat16)
    with guard_outputs("cpu"):
        y = ops.linear(x, w)                            # the PyTorch restatement stays inside its outputs as well
    assert y.shape == (5, 48)


@pytest.mark.gpu
def test_kernels_keep_inside_their_outputs_on_ragged_shapes():
    """GEMV, tcgen05 GEMM (token counts that do not fill a tile, output widths that do not fill a row tile), grouped MoE, norms,
    router, sampler and paged decode write only what they own."""
    from metal_marlin_b200 import ops
    from metal_marlin_b200.models.mmfp4_causal_lm import MMFP4ForCausalLM
    from metal_marlin_b200.ops import FP4Weight
    dev = "cuda"
    torch.manual_seed(0)
    for n_out, k in ((200, 256), (1344, 512), (72, 128)):
        w = FP4Weight.from_float(torch.randn(n_out, k, device=dev) * 0.05, 64)
        nw = torch.ones(k, dtype=torch.bfloat16, device=dev)
        for m in (1, 7, 33, 130, 300):
            x = (torch.randn(m, k, device=dev) * 0.5).to(torch.bfloat16)
            with guard_outputs(dev):
                y = ops.linear(x, w, norm_w=nw)
    lm = MMFP4ForCausalLM.from_config("tiny-mla-moe", device=dev, seed=1)
    for prompts in ([[5, 9, 2]], [list(range(1, 71)), [4, 4, 4, 4, 4]], [list(range(1, 300))]):
        with guard_outputs(dev):
            out = lm.generate(prompts, max_new_tokens=3, use_graph=False)
        assert all(len(o) == 3 for o in out)
    lm2 = MMFP4ForCausalLM.from_config("tiny-llama", device=dev, seed=1)
    with guard_outputs(dev):
        out = lm2.generate([list(range(1, 50)), [7]], max_new_tokens=3, use_graph=False)
    assert ops.check_status(torch.device(dev)) == 0
